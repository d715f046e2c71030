* c7552 (c7552: 32-bit adder / comparator): 416 gates, 3438 transistors
VDD vdd 0 DC 1.8
VIN0 na0 0 PULSE(0 1.8 5e-10 20p 20p 1e-09 2e-09)
VIN1 na1 0 PULSE(0 1.8 1e-09 20p 20p 2e-09 4e-09)
VIN2 na2 0 PULSE(0 1.8 2e-09 20p 20p 4e-09 8e-09)
VIN3 na3 0 PULSE(0 1.8 4e-09 20p 20p 8e-09 1.6e-08)
VIN4 na4 0 PULSE(0 1.8 8e-09 20p 20p 1.6e-08 3.2e-08)
VIN5 na5 0 PULSE(0 1.8 1.6e-08 20p 20p 3.2e-08 6.4e-08)
VIN6 na6 0 PULSE(0 1.8 3.2e-08 20p 20p 6.4e-08 1.28e-07)
VIN7 na7 0 PULSE(0 1.8 6.4e-08 20p 20p 1.28e-07 2.56e-07)
VIN8 na8 0 PULSE(0 1.8 1.28e-07 20p 20p 2.56e-07 5.12e-07)
VIN9 na9 0 PULSE(0 1.8 2.56e-07 20p 20p 5.12e-07 1.024e-06)
VIN10 na10 0 PULSE(0 1.8 5.12e-07 20p 20p 1.024e-06 2.048e-06)
VIN11 na11 0 PULSE(0 1.8 1.024e-06 20p 20p 2.048e-06 4.096e-06)
VIN12 na12 0 PULSE(0 1.8 2.048e-06 20p 20p 4.096e-06 8.192e-06)
VIN13 na13 0 PULSE(0 1.8 4.096e-06 20p 20p 8.192e-06 1.6384e-05)
VIN14 na14 0 PULSE(0 1.8 8.192e-06 20p 20p 1.6384e-05 3.2768e-05)
VIN15 na15 0 PULSE(0 1.8 1.6384e-05 20p 20p 3.2768e-05 6.5536e-05)
VIN16 na16 0 PULSE(0 1.8 3.2768e-05 20p 20p 6.5536e-05 0.000131072)
VIN17 na17 0 PULSE(0 1.8 6.5536e-05 20p 20p 0.000131072 0.000262144)
VIN18 na18 0 PULSE(0 1.8 0.000131072 20p 20p 0.000262144 0.000524288)
VIN19 na19 0 PULSE(0 1.8 0.000262144 20p 20p 0.000524288 0.001048576)
VIN20 na20 0 PULSE(0 1.8 0.000524288 20p 20p 0.001048576 0.002097152)
VIN21 na21 0 PULSE(0 1.8 0.001048576 20p 20p 0.002097152 0.004194304)
VIN22 na22 0 PULSE(0 1.8 0.002097152 20p 20p 0.004194304 0.008388608)
VIN23 na23 0 PULSE(0 1.8 0.004194304 20p 20p 0.008388608 0.016777216)
VIN24 na24 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN25 na25 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN26 na26 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN27 na27 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN28 na28 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN29 na29 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN30 na30 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN31 na31 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN32 nb0 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN33 nb1 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN34 nb2 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN35 nb3 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN36 nb4 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN37 nb5 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN38 nb6 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN39 nb7 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN40 nb8 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN41 nb9 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN42 nb10 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN43 nb11 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN44 nb12 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN45 nb13 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN46 nb14 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN47 nb15 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN48 nb16 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN49 nb17 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN50 nb18 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN51 nb19 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN52 nb20 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN53 nb21 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN54 nb22 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN55 nb23 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN56 nb24 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN57 nb25 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN58 nb26 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN59 nb27 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN60 nb28 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN61 nb29 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN62 nb30 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN63 nb31 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN64 ncin 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
CT1 t1 0 0.1f
CT2 t2 0 0.1f
CT3 t3 0 0.1f
M1 t1 na0 vdd vdd pch w=2u l=180n
M2 t1 nb0 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M3 t1 na0 t4 0 nch w=1u l=180n
M4 t4 nb0 0 0 nch w=1u l=180n
M5 t2 na0 vdd vdd pch w=2u l=180n
M6 t2 t1 vdd vdd pch w=2u l=180n
CT5 t5 0 0.1f
M7 t2 na0 t5 0 nch w=1u l=180n
M8 t5 t1 0 0 nch w=1u l=180n
M9 t3 nb0 vdd vdd pch w=2u l=180n
M10 t3 t1 vdd vdd pch w=2u l=180n
CT6 t6 0 0.1f
M11 t3 nb0 t6 0 nch w=1u l=180n
M12 t6 t1 0 0 nch w=1u l=180n
M13 nw1 t2 vdd vdd pch w=2u l=180n
M14 nw1 t3 vdd vdd pch w=2u l=180n
CT7 t7 0 0.1f
M15 nw1 t2 t7 0 nch w=1u l=180n
M16 t7 t3 0 0 nch w=1u l=180n
Cnw1 nw1 0 2f
CT8 t8 0 0.1f
CT9 t9 0 0.1f
CT10 t10 0 0.1f
M17 t8 nw1 vdd vdd pch w=2u l=180n
M18 t8 ncin vdd vdd pch w=2u l=180n
CT11 t11 0 0.1f
M19 t8 nw1 t11 0 nch w=1u l=180n
M20 t11 ncin 0 0 nch w=1u l=180n
M21 t9 nw1 vdd vdd pch w=2u l=180n
M22 t9 t8 vdd vdd pch w=2u l=180n
CT12 t12 0 0.1f
M23 t9 nw1 t12 0 nch w=1u l=180n
M24 t12 t8 0 0 nch w=1u l=180n
M25 t10 ncin vdd vdd pch w=2u l=180n
M26 t10 t8 vdd vdd pch w=2u l=180n
CT13 t13 0 0.1f
M27 t10 ncin t13 0 nch w=1u l=180n
M28 t13 t8 0 0 nch w=1u l=180n
M29 nw2 t9 vdd vdd pch w=2u l=180n
M30 nw2 t10 vdd vdd pch w=2u l=180n
CT14 t14 0 0.1f
M31 nw2 t9 t14 0 nch w=1u l=180n
M32 t14 t10 0 0 nch w=1u l=180n
Cnw2 nw2 0 2f
M33 nw3 na0 vdd vdd pch w=2u l=180n
M34 nw3 nb0 vdd vdd pch w=2u l=180n
CT15 t15 0 0.1f
M35 nw3 na0 t15 0 nch w=1u l=180n
M36 t15 nb0 0 0 nch w=1u l=180n
Cnw3 nw3 0 2f
M37 nw4 nw1 vdd vdd pch w=2u l=180n
M38 nw4 ncin vdd vdd pch w=2u l=180n
CT16 t16 0 0.1f
M39 nw4 nw1 t16 0 nch w=1u l=180n
M40 t16 ncin 0 0 nch w=1u l=180n
Cnw4 nw4 0 2f
M41 nw5 nw3 vdd vdd pch w=2u l=180n
M42 nw5 nw4 vdd vdd pch w=2u l=180n
CT17 t17 0 0.1f
M43 nw5 nw3 t17 0 nch w=1u l=180n
M44 t17 nw4 0 0 nch w=1u l=180n
Cnw5 nw5 0 2f
CT18 t18 0 0.1f
M45 t18 nw2 vdd vdd pch w=2u l=180n
M46 t18 nw2 0 0 nch w=1u l=180n
M47 ns0 t18 vdd vdd pch w=2u l=180n
M48 ns0 t18 0 0 nch w=1u l=180n
Cns0 ns0 0 2f
CT19 t19 0 0.1f
CT20 t20 0 0.1f
CT21 t21 0 0.1f
M49 t19 na1 vdd vdd pch w=2u l=180n
M50 t19 nb1 vdd vdd pch w=2u l=180n
CT22 t22 0 0.1f
M51 t19 na1 t22 0 nch w=1u l=180n
M52 t22 nb1 0 0 nch w=1u l=180n
M53 t20 na1 vdd vdd pch w=2u l=180n
M54 t20 t19 vdd vdd pch w=2u l=180n
CT23 t23 0 0.1f
M55 t20 na1 t23 0 nch w=1u l=180n
M56 t23 t19 0 0 nch w=1u l=180n
M57 t21 nb1 vdd vdd pch w=2u l=180n
M58 t21 t19 vdd vdd pch w=2u l=180n
CT24 t24 0 0.1f
M59 t21 nb1 t24 0 nch w=1u l=180n
M60 t24 t19 0 0 nch w=1u l=180n
M61 nw7 t20 vdd vdd pch w=2u l=180n
M62 nw7 t21 vdd vdd pch w=2u l=180n
CT25 t25 0 0.1f
M63 nw7 t20 t25 0 nch w=1u l=180n
M64 t25 t21 0 0 nch w=1u l=180n
Cnw7 nw7 0 2f
CT26 t26 0 0.1f
CT27 t27 0 0.1f
CT28 t28 0 0.1f
M65 t26 nw7 vdd vdd pch w=2u l=180n
M66 t26 nw5 vdd vdd pch w=2u l=180n
CT29 t29 0 0.1f
M67 t26 nw7 t29 0 nch w=1u l=180n
M68 t29 nw5 0 0 nch w=1u l=180n
M69 t27 nw7 vdd vdd pch w=2u l=180n
M70 t27 t26 vdd vdd pch w=2u l=180n
CT30 t30 0 0.1f
M71 t27 nw7 t30 0 nch w=1u l=180n
M72 t30 t26 0 0 nch w=1u l=180n
M73 t28 nw5 vdd vdd pch w=2u l=180n
M74 t28 t26 vdd vdd pch w=2u l=180n
CT31 t31 0 0.1f
M75 t28 nw5 t31 0 nch w=1u l=180n
M76 t31 t26 0 0 nch w=1u l=180n
M77 nw8 t27 vdd vdd pch w=2u l=180n
M78 nw8 t28 vdd vdd pch w=2u l=180n
CT32 t32 0 0.1f
M79 nw8 t27 t32 0 nch w=1u l=180n
M80 t32 t28 0 0 nch w=1u l=180n
Cnw8 nw8 0 2f
M81 nw9 na1 vdd vdd pch w=2u l=180n
M82 nw9 nb1 vdd vdd pch w=2u l=180n
CT33 t33 0 0.1f
M83 nw9 na1 t33 0 nch w=1u l=180n
M84 t33 nb1 0 0 nch w=1u l=180n
Cnw9 nw9 0 2f
M85 nw10 nw7 vdd vdd pch w=2u l=180n
M86 nw10 nw5 vdd vdd pch w=2u l=180n
CT34 t34 0 0.1f
M87 nw10 nw7 t34 0 nch w=1u l=180n
M88 t34 nw5 0 0 nch w=1u l=180n
Cnw10 nw10 0 2f
M89 nw11 nw9 vdd vdd pch w=2u l=180n
M90 nw11 nw10 vdd vdd pch w=2u l=180n
CT35 t35 0 0.1f
M91 nw11 nw9 t35 0 nch w=1u l=180n
M92 t35 nw10 0 0 nch w=1u l=180n
Cnw11 nw11 0 2f
CT36 t36 0 0.1f
M93 t36 nw8 vdd vdd pch w=2u l=180n
M94 t36 nw8 0 0 nch w=1u l=180n
M95 ns1 t36 vdd vdd pch w=2u l=180n
M96 ns1 t36 0 0 nch w=1u l=180n
Cns1 ns1 0 2f
CT37 t37 0 0.1f
CT38 t38 0 0.1f
CT39 t39 0 0.1f
M97 t37 nw2 vdd vdd pch w=2u l=180n
M98 t37 nw8 vdd vdd pch w=2u l=180n
CT40 t40 0 0.1f
M99 t37 nw2 t40 0 nch w=1u l=180n
M100 t40 nw8 0 0 nch w=1u l=180n
M101 t38 nw2 vdd vdd pch w=2u l=180n
M102 t38 t37 vdd vdd pch w=2u l=180n
CT41 t41 0 0.1f
M103 t38 nw2 t41 0 nch w=1u l=180n
M104 t41 t37 0 0 nch w=1u l=180n
M105 t39 nw8 vdd vdd pch w=2u l=180n
M106 t39 t37 vdd vdd pch w=2u l=180n
CT42 t42 0 0.1f
M107 t39 nw8 t42 0 nch w=1u l=180n
M108 t42 t37 0 0 nch w=1u l=180n
M109 nw13 t38 vdd vdd pch w=2u l=180n
M110 nw13 t39 vdd vdd pch w=2u l=180n
CT43 t43 0 0.1f
M111 nw13 t38 t43 0 nch w=1u l=180n
M112 t43 t39 0 0 nch w=1u l=180n
Cnw13 nw13 0 2f
CT44 t44 0 0.1f
CT45 t45 0 0.1f
CT46 t46 0 0.1f
M113 t44 na2 vdd vdd pch w=2u l=180n
M114 t44 nb2 vdd vdd pch w=2u l=180n
CT47 t47 0 0.1f
M115 t44 na2 t47 0 nch w=1u l=180n
M116 t47 nb2 0 0 nch w=1u l=180n
M117 t45 na2 vdd vdd pch w=2u l=180n
M118 t45 t44 vdd vdd pch w=2u l=180n
CT48 t48 0 0.1f
M119 t45 na2 t48 0 nch w=1u l=180n
M120 t48 t44 0 0 nch w=1u l=180n
M121 t46 nb2 vdd vdd pch w=2u l=180n
M122 t46 t44 vdd vdd pch w=2u l=180n
CT49 t49 0 0.1f
M123 t46 nb2 t49 0 nch w=1u l=180n
M124 t49 t44 0 0 nch w=1u l=180n
M125 nw14 t45 vdd vdd pch w=2u l=180n
M126 nw14 t46 vdd vdd pch w=2u l=180n
CT50 t50 0 0.1f
M127 nw14 t45 t50 0 nch w=1u l=180n
M128 t50 t46 0 0 nch w=1u l=180n
Cnw14 nw14 0 2f
CT51 t51 0 0.1f
CT52 t52 0 0.1f
CT53 t53 0 0.1f
M129 t51 nw14 vdd vdd pch w=2u l=180n
M130 t51 nw11 vdd vdd pch w=2u l=180n
CT54 t54 0 0.1f
M131 t51 nw14 t54 0 nch w=1u l=180n
M132 t54 nw11 0 0 nch w=1u l=180n
M133 t52 nw14 vdd vdd pch w=2u l=180n
M134 t52 t51 vdd vdd pch w=2u l=180n
CT55 t55 0 0.1f
M135 t52 nw14 t55 0 nch w=1u l=180n
M136 t55 t51 0 0 nch w=1u l=180n
M137 t53 nw11 vdd vdd pch w=2u l=180n
M138 t53 t51 vdd vdd pch w=2u l=180n
CT56 t56 0 0.1f
M139 t53 nw11 t56 0 nch w=1u l=180n
M140 t56 t51 0 0 nch w=1u l=180n
M141 nw15 t52 vdd vdd pch w=2u l=180n
M142 nw15 t53 vdd vdd pch w=2u l=180n
CT57 t57 0 0.1f
M143 nw15 t52 t57 0 nch w=1u l=180n
M144 t57 t53 0 0 nch w=1u l=180n
Cnw15 nw15 0 2f
M145 nw16 na2 vdd vdd pch w=2u l=180n
M146 nw16 nb2 vdd vdd pch w=2u l=180n
CT58 t58 0 0.1f
M147 nw16 na2 t58 0 nch w=1u l=180n
M148 t58 nb2 0 0 nch w=1u l=180n
Cnw16 nw16 0 2f
M149 nw17 nw14 vdd vdd pch w=2u l=180n
M150 nw17 nw11 vdd vdd pch w=2u l=180n
CT59 t59 0 0.1f
M151 nw17 nw14 t59 0 nch w=1u l=180n
M152 t59 nw11 0 0 nch w=1u l=180n
Cnw17 nw17 0 2f
M153 nw18 nw16 vdd vdd pch w=2u l=180n
M154 nw18 nw17 vdd vdd pch w=2u l=180n
CT60 t60 0 0.1f
M155 nw18 nw16 t60 0 nch w=1u l=180n
M156 t60 nw17 0 0 nch w=1u l=180n
Cnw18 nw18 0 2f
CT61 t61 0 0.1f
M157 t61 nw15 vdd vdd pch w=2u l=180n
M158 t61 nw15 0 0 nch w=1u l=180n
M159 ns2 t61 vdd vdd pch w=2u l=180n
M160 ns2 t61 0 0 nch w=1u l=180n
Cns2 ns2 0 2f
CT62 t62 0 0.1f
CT63 t63 0 0.1f
CT64 t64 0 0.1f
M161 t62 nw13 vdd vdd pch w=2u l=180n
M162 t62 nw15 vdd vdd pch w=2u l=180n
CT65 t65 0 0.1f
M163 t62 nw13 t65 0 nch w=1u l=180n
M164 t65 nw15 0 0 nch w=1u l=180n
M165 t63 nw13 vdd vdd pch w=2u l=180n
M166 t63 t62 vdd vdd pch w=2u l=180n
CT66 t66 0 0.1f
M167 t63 nw13 t66 0 nch w=1u l=180n
M168 t66 t62 0 0 nch w=1u l=180n
M169 t64 nw15 vdd vdd pch w=2u l=180n
M170 t64 t62 vdd vdd pch w=2u l=180n
CT67 t67 0 0.1f
M171 t64 nw15 t67 0 nch w=1u l=180n
M172 t67 t62 0 0 nch w=1u l=180n
M173 nw20 t63 vdd vdd pch w=2u l=180n
M174 nw20 t64 vdd vdd pch w=2u l=180n
CT68 t68 0 0.1f
M175 nw20 t63 t68 0 nch w=1u l=180n
M176 t68 t64 0 0 nch w=1u l=180n
Cnw20 nw20 0 2f
CT69 t69 0 0.1f
CT70 t70 0 0.1f
CT71 t71 0 0.1f
M177 t69 na3 vdd vdd pch w=2u l=180n
M178 t69 nb3 vdd vdd pch w=2u l=180n
CT72 t72 0 0.1f
M179 t69 na3 t72 0 nch w=1u l=180n
M180 t72 nb3 0 0 nch w=1u l=180n
M181 t70 na3 vdd vdd pch w=2u l=180n
M182 t70 t69 vdd vdd pch w=2u l=180n
CT73 t73 0 0.1f
M183 t70 na3 t73 0 nch w=1u l=180n
M184 t73 t69 0 0 nch w=1u l=180n
M185 t71 nb3 vdd vdd pch w=2u l=180n
M186 t71 t69 vdd vdd pch w=2u l=180n
CT74 t74 0 0.1f
M187 t71 nb3 t74 0 nch w=1u l=180n
M188 t74 t69 0 0 nch w=1u l=180n
M189 nw21 t70 vdd vdd pch w=2u l=180n
M190 nw21 t71 vdd vdd pch w=2u l=180n
CT75 t75 0 0.1f
M191 nw21 t70 t75 0 nch w=1u l=180n
M192 t75 t71 0 0 nch w=1u l=180n
Cnw21 nw21 0 2f
CT76 t76 0 0.1f
CT77 t77 0 0.1f
CT78 t78 0 0.1f
M193 t76 nw21 vdd vdd pch w=2u l=180n
M194 t76 nw18 vdd vdd pch w=2u l=180n
CT79 t79 0 0.1f
M195 t76 nw21 t79 0 nch w=1u l=180n
M196 t79 nw18 0 0 nch w=1u l=180n
M197 t77 nw21 vdd vdd pch w=2u l=180n
M198 t77 t76 vdd vdd pch w=2u l=180n
CT80 t80 0 0.1f
M199 t77 nw21 t80 0 nch w=1u l=180n
M200 t80 t76 0 0 nch w=1u l=180n
M201 t78 nw18 vdd vdd pch w=2u l=180n
M202 t78 t76 vdd vdd pch w=2u l=180n
CT81 t81 0 0.1f
M203 t78 nw18 t81 0 nch w=1u l=180n
M204 t81 t76 0 0 nch w=1u l=180n
M205 nw22 t77 vdd vdd pch w=2u l=180n
M206 nw22 t78 vdd vdd pch w=2u l=180n
CT82 t82 0 0.1f
M207 nw22 t77 t82 0 nch w=1u l=180n
M208 t82 t78 0 0 nch w=1u l=180n
Cnw22 nw22 0 2f
M209 nw23 na3 vdd vdd pch w=2u l=180n
M210 nw23 nb3 vdd vdd pch w=2u l=180n
CT83 t83 0 0.1f
M211 nw23 na3 t83 0 nch w=1u l=180n
M212 t83 nb3 0 0 nch w=1u l=180n
Cnw23 nw23 0 2f
M213 nw24 nw21 vdd vdd pch w=2u l=180n
M214 nw24 nw18 vdd vdd pch w=2u l=180n
CT84 t84 0 0.1f
M215 nw24 nw21 t84 0 nch w=1u l=180n
M216 t84 nw18 0 0 nch w=1u l=180n
Cnw24 nw24 0 2f
M217 nw25 nw23 vdd vdd pch w=2u l=180n
M218 nw25 nw24 vdd vdd pch w=2u l=180n
CT85 t85 0 0.1f
M219 nw25 nw23 t85 0 nch w=1u l=180n
M220 t85 nw24 0 0 nch w=1u l=180n
Cnw25 nw25 0 2f
CT86 t86 0 0.1f
M221 t86 nw22 vdd vdd pch w=2u l=180n
M222 t86 nw22 0 0 nch w=1u l=180n
M223 ns3 t86 vdd vdd pch w=2u l=180n
M224 ns3 t86 0 0 nch w=1u l=180n
Cns3 ns3 0 2f
CT87 t87 0 0.1f
CT88 t88 0 0.1f
CT89 t89 0 0.1f
M225 t87 nw20 vdd vdd pch w=2u l=180n
M226 t87 nw22 vdd vdd pch w=2u l=180n
CT90 t90 0 0.1f
M227 t87 nw20 t90 0 nch w=1u l=180n
M228 t90 nw22 0 0 nch w=1u l=180n
M229 t88 nw20 vdd vdd pch w=2u l=180n
M230 t88 t87 vdd vdd pch w=2u l=180n
CT91 t91 0 0.1f
M231 t88 nw20 t91 0 nch w=1u l=180n
M232 t91 t87 0 0 nch w=1u l=180n
M233 t89 nw22 vdd vdd pch w=2u l=180n
M234 t89 t87 vdd vdd pch w=2u l=180n
CT92 t92 0 0.1f
M235 t89 nw22 t92 0 nch w=1u l=180n
M236 t92 t87 0 0 nch w=1u l=180n
M237 nw27 t88 vdd vdd pch w=2u l=180n
M238 nw27 t89 vdd vdd pch w=2u l=180n
CT93 t93 0 0.1f
M239 nw27 t88 t93 0 nch w=1u l=180n
M240 t93 t89 0 0 nch w=1u l=180n
Cnw27 nw27 0 2f
CT94 t94 0 0.1f
CT95 t95 0 0.1f
CT96 t96 0 0.1f
M241 t94 na4 vdd vdd pch w=2u l=180n
M242 t94 nb4 vdd vdd pch w=2u l=180n
CT97 t97 0 0.1f
M243 t94 na4 t97 0 nch w=1u l=180n
M244 t97 nb4 0 0 nch w=1u l=180n
M245 t95 na4 vdd vdd pch w=2u l=180n
M246 t95 t94 vdd vdd pch w=2u l=180n
CT98 t98 0 0.1f
M247 t95 na4 t98 0 nch w=1u l=180n
M248 t98 t94 0 0 nch w=1u l=180n
M249 t96 nb4 vdd vdd pch w=2u l=180n
M250 t96 t94 vdd vdd pch w=2u l=180n
CT99 t99 0 0.1f
M251 t96 nb4 t99 0 nch w=1u l=180n
M252 t99 t94 0 0 nch w=1u l=180n
M253 nw28 t95 vdd vdd pch w=2u l=180n
M254 nw28 t96 vdd vdd pch w=2u l=180n
CT100 t100 0 0.1f
M255 nw28 t95 t100 0 nch w=1u l=180n
M256 t100 t96 0 0 nch w=1u l=180n
Cnw28 nw28 0 2f
CT101 t101 0 0.1f
CT102 t102 0 0.1f
CT103 t103 0 0.1f
M257 t101 nw28 vdd vdd pch w=2u l=180n
M258 t101 nw25 vdd vdd pch w=2u l=180n
CT104 t104 0 0.1f
M259 t101 nw28 t104 0 nch w=1u l=180n
M260 t104 nw25 0 0 nch w=1u l=180n
M261 t102 nw28 vdd vdd pch w=2u l=180n
M262 t102 t101 vdd vdd pch w=2u l=180n
CT105 t105 0 0.1f
M263 t102 nw28 t105 0 nch w=1u l=180n
M264 t105 t101 0 0 nch w=1u l=180n
M265 t103 nw25 vdd vdd pch w=2u l=180n
M266 t103 t101 vdd vdd pch w=2u l=180n
CT106 t106 0 0.1f
M267 t103 nw25 t106 0 nch w=1u l=180n
M268 t106 t101 0 0 nch w=1u l=180n
M269 nw29 t102 vdd vdd pch w=2u l=180n
M270 nw29 t103 vdd vdd pch w=2u l=180n
CT107 t107 0 0.1f
M271 nw29 t102 t107 0 nch w=1u l=180n
M272 t107 t103 0 0 nch w=1u l=180n
Cnw29 nw29 0 2f
M273 nw30 na4 vdd vdd pch w=2u l=180n
M274 nw30 nb4 vdd vdd pch w=2u l=180n
CT108 t108 0 0.1f
M275 nw30 na4 t108 0 nch w=1u l=180n
M276 t108 nb4 0 0 nch w=1u l=180n
Cnw30 nw30 0 2f
M277 nw31 nw28 vdd vdd pch w=2u l=180n
M278 nw31 nw25 vdd vdd pch w=2u l=180n
CT109 t109 0 0.1f
M279 nw31 nw28 t109 0 nch w=1u l=180n
M280 t109 nw25 0 0 nch w=1u l=180n
Cnw31 nw31 0 2f
M281 nw32 nw30 vdd vdd pch w=2u l=180n
M282 nw32 nw31 vdd vdd pch w=2u l=180n
CT110 t110 0 0.1f
M283 nw32 nw30 t110 0 nch w=1u l=180n
M284 t110 nw31 0 0 nch w=1u l=180n
Cnw32 nw32 0 2f
CT111 t111 0 0.1f
M285 t111 nw29 vdd vdd pch w=2u l=180n
M286 t111 nw29 0 0 nch w=1u l=180n
M287 ns4 t111 vdd vdd pch w=2u l=180n
M288 ns4 t111 0 0 nch w=1u l=180n
Cns4 ns4 0 2f
CT112 t112 0 0.1f
CT113 t113 0 0.1f
CT114 t114 0 0.1f
M289 t112 nw27 vdd vdd pch w=2u l=180n
M290 t112 nw29 vdd vdd pch w=2u l=180n
CT115 t115 0 0.1f
M291 t112 nw27 t115 0 nch w=1u l=180n
M292 t115 nw29 0 0 nch w=1u l=180n
M293 t113 nw27 vdd vdd pch w=2u l=180n
M294 t113 t112 vdd vdd pch w=2u l=180n
CT116 t116 0 0.1f
M295 t113 nw27 t116 0 nch w=1u l=180n
M296 t116 t112 0 0 nch w=1u l=180n
M297 t114 nw29 vdd vdd pch w=2u l=180n
M298 t114 t112 vdd vdd pch w=2u l=180n
CT117 t117 0 0.1f
M299 t114 nw29 t117 0 nch w=1u l=180n
M300 t117 t112 0 0 nch w=1u l=180n
M301 nw34 t113 vdd vdd pch w=2u l=180n
M302 nw34 t114 vdd vdd pch w=2u l=180n
CT118 t118 0 0.1f
M303 nw34 t113 t118 0 nch w=1u l=180n
M304 t118 t114 0 0 nch w=1u l=180n
Cnw34 nw34 0 2f
CT119 t119 0 0.1f
CT120 t120 0 0.1f
CT121 t121 0 0.1f
M305 t119 na5 vdd vdd pch w=2u l=180n
M306 t119 nb5 vdd vdd pch w=2u l=180n
CT122 t122 0 0.1f
M307 t119 na5 t122 0 nch w=1u l=180n
M308 t122 nb5 0 0 nch w=1u l=180n
M309 t120 na5 vdd vdd pch w=2u l=180n
M310 t120 t119 vdd vdd pch w=2u l=180n
CT123 t123 0 0.1f
M311 t120 na5 t123 0 nch w=1u l=180n
M312 t123 t119 0 0 nch w=1u l=180n
M313 t121 nb5 vdd vdd pch w=2u l=180n
M314 t121 t119 vdd vdd pch w=2u l=180n
CT124 t124 0 0.1f
M315 t121 nb5 t124 0 nch w=1u l=180n
M316 t124 t119 0 0 nch w=1u l=180n
M317 nw35 t120 vdd vdd pch w=2u l=180n
M318 nw35 t121 vdd vdd pch w=2u l=180n
CT125 t125 0 0.1f
M319 nw35 t120 t125 0 nch w=1u l=180n
M320 t125 t121 0 0 nch w=1u l=180n
Cnw35 nw35 0 2f
CT126 t126 0 0.1f
CT127 t127 0 0.1f
CT128 t128 0 0.1f
M321 t126 nw35 vdd vdd pch w=2u l=180n
M322 t126 nw32 vdd vdd pch w=2u l=180n
CT129 t129 0 0.1f
M323 t126 nw35 t129 0 nch w=1u l=180n
M324 t129 nw32 0 0 nch w=1u l=180n
M325 t127 nw35 vdd vdd pch w=2u l=180n
M326 t127 t126 vdd vdd pch w=2u l=180n
CT130 t130 0 0.1f
M327 t127 nw35 t130 0 nch w=1u l=180n
M328 t130 t126 0 0 nch w=1u l=180n
M329 t128 nw32 vdd vdd pch w=2u l=180n
M330 t128 t126 vdd vdd pch w=2u l=180n
CT131 t131 0 0.1f
M331 t128 nw32 t131 0 nch w=1u l=180n
M332 t131 t126 0 0 nch w=1u l=180n
M333 nw36 t127 vdd vdd pch w=2u l=180n
M334 nw36 t128 vdd vdd pch w=2u l=180n
CT132 t132 0 0.1f
M335 nw36 t127 t132 0 nch w=1u l=180n
M336 t132 t128 0 0 nch w=1u l=180n
Cnw36 nw36 0 2f
M337 nw37 na5 vdd vdd pch w=2u l=180n
M338 nw37 nb5 vdd vdd pch w=2u l=180n
CT133 t133 0 0.1f
M339 nw37 na5 t133 0 nch w=1u l=180n
M340 t133 nb5 0 0 nch w=1u l=180n
Cnw37 nw37 0 2f
M341 nw38 nw35 vdd vdd pch w=2u l=180n
M342 nw38 nw32 vdd vdd pch w=2u l=180n
CT134 t134 0 0.1f
M343 nw38 nw35 t134 0 nch w=1u l=180n
M344 t134 nw32 0 0 nch w=1u l=180n
Cnw38 nw38 0 2f
M345 nw39 nw37 vdd vdd pch w=2u l=180n
M346 nw39 nw38 vdd vdd pch w=2u l=180n
CT135 t135 0 0.1f
M347 nw39 nw37 t135 0 nch w=1u l=180n
M348 t135 nw38 0 0 nch w=1u l=180n
Cnw39 nw39 0 2f
CT136 t136 0 0.1f
M349 t136 nw36 vdd vdd pch w=2u l=180n
M350 t136 nw36 0 0 nch w=1u l=180n
M351 ns5 t136 vdd vdd pch w=2u l=180n
M352 ns5 t136 0 0 nch w=1u l=180n
Cns5 ns5 0 2f
CT137 t137 0 0.1f
CT138 t138 0 0.1f
CT139 t139 0 0.1f
M353 t137 nw34 vdd vdd pch w=2u l=180n
M354 t137 nw36 vdd vdd pch w=2u l=180n
CT140 t140 0 0.1f
M355 t137 nw34 t140 0 nch w=1u l=180n
M356 t140 nw36 0 0 nch w=1u l=180n
M357 t138 nw34 vdd vdd pch w=2u l=180n
M358 t138 t137 vdd vdd pch w=2u l=180n
CT141 t141 0 0.1f
M359 t138 nw34 t141 0 nch w=1u l=180n
M360 t141 t137 0 0 nch w=1u l=180n
M361 t139 nw36 vdd vdd pch w=2u l=180n
M362 t139 t137 vdd vdd pch w=2u l=180n
CT142 t142 0 0.1f
M363 t139 nw36 t142 0 nch w=1u l=180n
M364 t142 t137 0 0 nch w=1u l=180n
M365 nw41 t138 vdd vdd pch w=2u l=180n
M366 nw41 t139 vdd vdd pch w=2u l=180n
CT143 t143 0 0.1f
M367 nw41 t138 t143 0 nch w=1u l=180n
M368 t143 t139 0 0 nch w=1u l=180n
Cnw41 nw41 0 2f
CT144 t144 0 0.1f
CT145 t145 0 0.1f
CT146 t146 0 0.1f
M369 t144 na6 vdd vdd pch w=2u l=180n
M370 t144 nb6 vdd vdd pch w=2u l=180n
CT147 t147 0 0.1f
M371 t144 na6 t147 0 nch w=1u l=180n
M372 t147 nb6 0 0 nch w=1u l=180n
M373 t145 na6 vdd vdd pch w=2u l=180n
M374 t145 t144 vdd vdd pch w=2u l=180n
CT148 t148 0 0.1f
M375 t145 na6 t148 0 nch w=1u l=180n
M376 t148 t144 0 0 nch w=1u l=180n
M377 t146 nb6 vdd vdd pch w=2u l=180n
M378 t146 t144 vdd vdd pch w=2u l=180n
CT149 t149 0 0.1f
M379 t146 nb6 t149 0 nch w=1u l=180n
M380 t149 t144 0 0 nch w=1u l=180n
M381 nw42 t145 vdd vdd pch w=2u l=180n
M382 nw42 t146 vdd vdd pch w=2u l=180n
CT150 t150 0 0.1f
M383 nw42 t145 t150 0 nch w=1u l=180n
M384 t150 t146 0 0 nch w=1u l=180n
Cnw42 nw42 0 2f
CT151 t151 0 0.1f
CT152 t152 0 0.1f
CT153 t153 0 0.1f
M385 t151 nw42 vdd vdd pch w=2u l=180n
M386 t151 nw39 vdd vdd pch w=2u l=180n
CT154 t154 0 0.1f
M387 t151 nw42 t154 0 nch w=1u l=180n
M388 t154 nw39 0 0 nch w=1u l=180n
M389 t152 nw42 vdd vdd pch w=2u l=180n
M390 t152 t151 vdd vdd pch w=2u l=180n
CT155 t155 0 0.1f
M391 t152 nw42 t155 0 nch w=1u l=180n
M392 t155 t151 0 0 nch w=1u l=180n
M393 t153 nw39 vdd vdd pch w=2u l=180n
M394 t153 t151 vdd vdd pch w=2u l=180n
CT156 t156 0 0.1f
M395 t153 nw39 t156 0 nch w=1u l=180n
M396 t156 t151 0 0 nch w=1u l=180n
M397 nw43 t152 vdd vdd pch w=2u l=180n
M398 nw43 t153 vdd vdd pch w=2u l=180n
CT157 t157 0 0.1f
M399 nw43 t152 t157 0 nch w=1u l=180n
M400 t157 t153 0 0 nch w=1u l=180n
Cnw43 nw43 0 2f
M401 nw44 na6 vdd vdd pch w=2u l=180n
M402 nw44 nb6 vdd vdd pch w=2u l=180n
CT158 t158 0 0.1f
M403 nw44 na6 t158 0 nch w=1u l=180n
M404 t158 nb6 0 0 nch w=1u l=180n
Cnw44 nw44 0 2f
M405 nw45 nw42 vdd vdd pch w=2u l=180n
M406 nw45 nw39 vdd vdd pch w=2u l=180n
CT159 t159 0 0.1f
M407 nw45 nw42 t159 0 nch w=1u l=180n
M408 t159 nw39 0 0 nch w=1u l=180n
Cnw45 nw45 0 2f
M409 nw46 nw44 vdd vdd pch w=2u l=180n
M410 nw46 nw45 vdd vdd pch w=2u l=180n
CT160 t160 0 0.1f
M411 nw46 nw44 t160 0 nch w=1u l=180n
M412 t160 nw45 0 0 nch w=1u l=180n
Cnw46 nw46 0 2f
CT161 t161 0 0.1f
M413 t161 nw43 vdd vdd pch w=2u l=180n
M414 t161 nw43 0 0 nch w=1u l=180n
M415 ns6 t161 vdd vdd pch w=2u l=180n
M416 ns6 t161 0 0 nch w=1u l=180n
Cns6 ns6 0 2f
CT162 t162 0 0.1f
CT163 t163 0 0.1f
CT164 t164 0 0.1f
M417 t162 nw41 vdd vdd pch w=2u l=180n
M418 t162 nw43 vdd vdd pch w=2u l=180n
CT165 t165 0 0.1f
M419 t162 nw41 t165 0 nch w=1u l=180n
M420 t165 nw43 0 0 nch w=1u l=180n
M421 t163 nw41 vdd vdd pch w=2u l=180n
M422 t163 t162 vdd vdd pch w=2u l=180n
CT166 t166 0 0.1f
M423 t163 nw41 t166 0 nch w=1u l=180n
M424 t166 t162 0 0 nch w=1u l=180n
M425 t164 nw43 vdd vdd pch w=2u l=180n
M426 t164 t162 vdd vdd pch w=2u l=180n
CT167 t167 0 0.1f
M427 t164 nw43 t167 0 nch w=1u l=180n
M428 t167 t162 0 0 nch w=1u l=180n
M429 nw48 t163 vdd vdd pch w=2u l=180n
M430 nw48 t164 vdd vdd pch w=2u l=180n
CT168 t168 0 0.1f
M431 nw48 t163 t168 0 nch w=1u l=180n
M432 t168 t164 0 0 nch w=1u l=180n
Cnw48 nw48 0 2f
CT169 t169 0 0.1f
CT170 t170 0 0.1f
CT171 t171 0 0.1f
M433 t169 na7 vdd vdd pch w=2u l=180n
M434 t169 nb7 vdd vdd pch w=2u l=180n
CT172 t172 0 0.1f
M435 t169 na7 t172 0 nch w=1u l=180n
M436 t172 nb7 0 0 nch w=1u l=180n
M437 t170 na7 vdd vdd pch w=2u l=180n
M438 t170 t169 vdd vdd pch w=2u l=180n
CT173 t173 0 0.1f
M439 t170 na7 t173 0 nch w=1u l=180n
M440 t173 t169 0 0 nch w=1u l=180n
M441 t171 nb7 vdd vdd pch w=2u l=180n
M442 t171 t169 vdd vdd pch w=2u l=180n
CT174 t174 0 0.1f
M443 t171 nb7 t174 0 nch w=1u l=180n
M444 t174 t169 0 0 nch w=1u l=180n
M445 nw49 t170 vdd vdd pch w=2u l=180n
M446 nw49 t171 vdd vdd pch w=2u l=180n
CT175 t175 0 0.1f
M447 nw49 t170 t175 0 nch w=1u l=180n
M448 t175 t171 0 0 nch w=1u l=180n
Cnw49 nw49 0 2f
CT176 t176 0 0.1f
CT177 t177 0 0.1f
CT178 t178 0 0.1f
M449 t176 nw49 vdd vdd pch w=2u l=180n
M450 t176 nw46 vdd vdd pch w=2u l=180n
CT179 t179 0 0.1f
M451 t176 nw49 t179 0 nch w=1u l=180n
M452 t179 nw46 0 0 nch w=1u l=180n
M453 t177 nw49 vdd vdd pch w=2u l=180n
M454 t177 t176 vdd vdd pch w=2u l=180n
CT180 t180 0 0.1f
M455 t177 nw49 t180 0 nch w=1u l=180n
M456 t180 t176 0 0 nch w=1u l=180n
M457 t178 nw46 vdd vdd pch w=2u l=180n
M458 t178 t176 vdd vdd pch w=2u l=180n
CT181 t181 0 0.1f
M459 t178 nw46 t181 0 nch w=1u l=180n
M460 t181 t176 0 0 nch w=1u l=180n
M461 nw50 t177 vdd vdd pch w=2u l=180n
M462 nw50 t178 vdd vdd pch w=2u l=180n
CT182 t182 0 0.1f
M463 nw50 t177 t182 0 nch w=1u l=180n
M464 t182 t178 0 0 nch w=1u l=180n
Cnw50 nw50 0 2f
M465 nw51 na7 vdd vdd pch w=2u l=180n
M466 nw51 nb7 vdd vdd pch w=2u l=180n
CT183 t183 0 0.1f
M467 nw51 na7 t183 0 nch w=1u l=180n
M468 t183 nb7 0 0 nch w=1u l=180n
Cnw51 nw51 0 2f
M469 nw52 nw49 vdd vdd pch w=2u l=180n
M470 nw52 nw46 vdd vdd pch w=2u l=180n
CT184 t184 0 0.1f
M471 nw52 nw49 t184 0 nch w=1u l=180n
M472 t184 nw46 0 0 nch w=1u l=180n
Cnw52 nw52 0 2f
M473 nw53 nw51 vdd vdd pch w=2u l=180n
M474 nw53 nw52 vdd vdd pch w=2u l=180n
CT185 t185 0 0.1f
M475 nw53 nw51 t185 0 nch w=1u l=180n
M476 t185 nw52 0 0 nch w=1u l=180n
Cnw53 nw53 0 2f
CT186 t186 0 0.1f
M477 t186 nw50 vdd vdd pch w=2u l=180n
M478 t186 nw50 0 0 nch w=1u l=180n
M479 ns7 t186 vdd vdd pch w=2u l=180n
M480 ns7 t186 0 0 nch w=1u l=180n
Cns7 ns7 0 2f
CT187 t187 0 0.1f
CT188 t188 0 0.1f
CT189 t189 0 0.1f
M481 t187 nw48 vdd vdd pch w=2u l=180n
M482 t187 nw50 vdd vdd pch w=2u l=180n
CT190 t190 0 0.1f
M483 t187 nw48 t190 0 nch w=1u l=180n
M484 t190 nw50 0 0 nch w=1u l=180n
M485 t188 nw48 vdd vdd pch w=2u l=180n
M486 t188 t187 vdd vdd pch w=2u l=180n
CT191 t191 0 0.1f
M487 t188 nw48 t191 0 nch w=1u l=180n
M488 t191 t187 0 0 nch w=1u l=180n
M489 t189 nw50 vdd vdd pch w=2u l=180n
M490 t189 t187 vdd vdd pch w=2u l=180n
CT192 t192 0 0.1f
M491 t189 nw50 t192 0 nch w=1u l=180n
M492 t192 t187 0 0 nch w=1u l=180n
M493 nw55 t188 vdd vdd pch w=2u l=180n
M494 nw55 t189 vdd vdd pch w=2u l=180n
CT193 t193 0 0.1f
M495 nw55 t188 t193 0 nch w=1u l=180n
M496 t193 t189 0 0 nch w=1u l=180n
Cnw55 nw55 0 2f
CT194 t194 0 0.1f
CT195 t195 0 0.1f
CT196 t196 0 0.1f
M497 t194 na8 vdd vdd pch w=2u l=180n
M498 t194 nb8 vdd vdd pch w=2u l=180n
CT197 t197 0 0.1f
M499 t194 na8 t197 0 nch w=1u l=180n
M500 t197 nb8 0 0 nch w=1u l=180n
M501 t195 na8 vdd vdd pch w=2u l=180n
M502 t195 t194 vdd vdd pch w=2u l=180n
CT198 t198 0 0.1f
M503 t195 na8 t198 0 nch w=1u l=180n
M504 t198 t194 0 0 nch w=1u l=180n
M505 t196 nb8 vdd vdd pch w=2u l=180n
M506 t196 t194 vdd vdd pch w=2u l=180n
CT199 t199 0 0.1f
M507 t196 nb8 t199 0 nch w=1u l=180n
M508 t199 t194 0 0 nch w=1u l=180n
M509 nw56 t195 vdd vdd pch w=2u l=180n
M510 nw56 t196 vdd vdd pch w=2u l=180n
CT200 t200 0 0.1f
M511 nw56 t195 t200 0 nch w=1u l=180n
M512 t200 t196 0 0 nch w=1u l=180n
Cnw56 nw56 0 2f
CT201 t201 0 0.1f
CT202 t202 0 0.1f
CT203 t203 0 0.1f
M513 t201 nw56 vdd vdd pch w=2u l=180n
M514 t201 nw53 vdd vdd pch w=2u l=180n
CT204 t204 0 0.1f
M515 t201 nw56 t204 0 nch w=1u l=180n
M516 t204 nw53 0 0 nch w=1u l=180n
M517 t202 nw56 vdd vdd pch w=2u l=180n
M518 t202 t201 vdd vdd pch w=2u l=180n
CT205 t205 0 0.1f
M519 t202 nw56 t205 0 nch w=1u l=180n
M520 t205 t201 0 0 nch w=1u l=180n
M521 t203 nw53 vdd vdd pch w=2u l=180n
M522 t203 t201 vdd vdd pch w=2u l=180n
CT206 t206 0 0.1f
M523 t203 nw53 t206 0 nch w=1u l=180n
M524 t206 t201 0 0 nch w=1u l=180n
M525 nw57 t202 vdd vdd pch w=2u l=180n
M526 nw57 t203 vdd vdd pch w=2u l=180n
CT207 t207 0 0.1f
M527 nw57 t202 t207 0 nch w=1u l=180n
M528 t207 t203 0 0 nch w=1u l=180n
Cnw57 nw57 0 2f
M529 nw58 na8 vdd vdd pch w=2u l=180n
M530 nw58 nb8 vdd vdd pch w=2u l=180n
CT208 t208 0 0.1f
M531 nw58 na8 t208 0 nch w=1u l=180n
M532 t208 nb8 0 0 nch w=1u l=180n
Cnw58 nw58 0 2f
M533 nw59 nw56 vdd vdd pch w=2u l=180n
M534 nw59 nw53 vdd vdd pch w=2u l=180n
CT209 t209 0 0.1f
M535 nw59 nw56 t209 0 nch w=1u l=180n
M536 t209 nw53 0 0 nch w=1u l=180n
Cnw59 nw59 0 2f
M537 nw60 nw58 vdd vdd pch w=2u l=180n
M538 nw60 nw59 vdd vdd pch w=2u l=180n
CT210 t210 0 0.1f
M539 nw60 nw58 t210 0 nch w=1u l=180n
M540 t210 nw59 0 0 nch w=1u l=180n
Cnw60 nw60 0 2f
CT211 t211 0 0.1f
M541 t211 nw57 vdd vdd pch w=2u l=180n
M542 t211 nw57 0 0 nch w=1u l=180n
M543 ns8 t211 vdd vdd pch w=2u l=180n
M544 ns8 t211 0 0 nch w=1u l=180n
Cns8 ns8 0 2f
CT212 t212 0 0.1f
CT213 t213 0 0.1f
CT214 t214 0 0.1f
M545 t212 nw55 vdd vdd pch w=2u l=180n
M546 t212 nw57 vdd vdd pch w=2u l=180n
CT215 t215 0 0.1f
M547 t212 nw55 t215 0 nch w=1u l=180n
M548 t215 nw57 0 0 nch w=1u l=180n
M549 t213 nw55 vdd vdd pch w=2u l=180n
M550 t213 t212 vdd vdd pch w=2u l=180n
CT216 t216 0 0.1f
M551 t213 nw55 t216 0 nch w=1u l=180n
M552 t216 t212 0 0 nch w=1u l=180n
M553 t214 nw57 vdd vdd pch w=2u l=180n
M554 t214 t212 vdd vdd pch w=2u l=180n
CT217 t217 0 0.1f
M555 t214 nw57 t217 0 nch w=1u l=180n
M556 t217 t212 0 0 nch w=1u l=180n
M557 nw62 t213 vdd vdd pch w=2u l=180n
M558 nw62 t214 vdd vdd pch w=2u l=180n
CT218 t218 0 0.1f
M559 nw62 t213 t218 0 nch w=1u l=180n
M560 t218 t214 0 0 nch w=1u l=180n
Cnw62 nw62 0 2f
CT219 t219 0 0.1f
CT220 t220 0 0.1f
CT221 t221 0 0.1f
M561 t219 na9 vdd vdd pch w=2u l=180n
M562 t219 nb9 vdd vdd pch w=2u l=180n
CT222 t222 0 0.1f
M563 t219 na9 t222 0 nch w=1u l=180n
M564 t222 nb9 0 0 nch w=1u l=180n
M565 t220 na9 vdd vdd pch w=2u l=180n
M566 t220 t219 vdd vdd pch w=2u l=180n
CT223 t223 0 0.1f
M567 t220 na9 t223 0 nch w=1u l=180n
M568 t223 t219 0 0 nch w=1u l=180n
M569 t221 nb9 vdd vdd pch w=2u l=180n
M570 t221 t219 vdd vdd pch w=2u l=180n
CT224 t224 0 0.1f
M571 t221 nb9 t224 0 nch w=1u l=180n
M572 t224 t219 0 0 nch w=1u l=180n
M573 nw63 t220 vdd vdd pch w=2u l=180n
M574 nw63 t221 vdd vdd pch w=2u l=180n
CT225 t225 0 0.1f
M575 nw63 t220 t225 0 nch w=1u l=180n
M576 t225 t221 0 0 nch w=1u l=180n
Cnw63 nw63 0 2f
CT226 t226 0 0.1f
CT227 t227 0 0.1f
CT228 t228 0 0.1f
M577 t226 nw63 vdd vdd pch w=2u l=180n
M578 t226 nw60 vdd vdd pch w=2u l=180n
CT229 t229 0 0.1f
M579 t226 nw63 t229 0 nch w=1u l=180n
M580 t229 nw60 0 0 nch w=1u l=180n
M581 t227 nw63 vdd vdd pch w=2u l=180n
M582 t227 t226 vdd vdd pch w=2u l=180n
CT230 t230 0 0.1f
M583 t227 nw63 t230 0 nch w=1u l=180n
M584 t230 t226 0 0 nch w=1u l=180n
M585 t228 nw60 vdd vdd pch w=2u l=180n
M586 t228 t226 vdd vdd pch w=2u l=180n
CT231 t231 0 0.1f
M587 t228 nw60 t231 0 nch w=1u l=180n
M588 t231 t226 0 0 nch w=1u l=180n
M589 nw64 t227 vdd vdd pch w=2u l=180n
M590 nw64 t228 vdd vdd pch w=2u l=180n
CT232 t232 0 0.1f
M591 nw64 t227 t232 0 nch w=1u l=180n
M592 t232 t228 0 0 nch w=1u l=180n
Cnw64 nw64 0 2f
M593 nw65 na9 vdd vdd pch w=2u l=180n
M594 nw65 nb9 vdd vdd pch w=2u l=180n
CT233 t233 0 0.1f
M595 nw65 na9 t233 0 nch w=1u l=180n
M596 t233 nb9 0 0 nch w=1u l=180n
Cnw65 nw65 0 2f
M597 nw66 nw63 vdd vdd pch w=2u l=180n
M598 nw66 nw60 vdd vdd pch w=2u l=180n
CT234 t234 0 0.1f
M599 nw66 nw63 t234 0 nch w=1u l=180n
M600 t234 nw60 0 0 nch w=1u l=180n
Cnw66 nw66 0 2f
M601 nw67 nw65 vdd vdd pch w=2u l=180n
M602 nw67 nw66 vdd vdd pch w=2u l=180n
CT235 t235 0 0.1f
M603 nw67 nw65 t235 0 nch w=1u l=180n
M604 t235 nw66 0 0 nch w=1u l=180n
Cnw67 nw67 0 2f
CT236 t236 0 0.1f
M605 t236 nw64 vdd vdd pch w=2u l=180n
M606 t236 nw64 0 0 nch w=1u l=180n
M607 ns9 t236 vdd vdd pch w=2u l=180n
M608 ns9 t236 0 0 nch w=1u l=180n
Cns9 ns9 0 2f
CT237 t237 0 0.1f
CT238 t238 0 0.1f
CT239 t239 0 0.1f
M609 t237 nw62 vdd vdd pch w=2u l=180n
M610 t237 nw64 vdd vdd pch w=2u l=180n
CT240 t240 0 0.1f
M611 t237 nw62 t240 0 nch w=1u l=180n
M612 t240 nw64 0 0 nch w=1u l=180n
M613 t238 nw62 vdd vdd pch w=2u l=180n
M614 t238 t237 vdd vdd pch w=2u l=180n
CT241 t241 0 0.1f
M615 t238 nw62 t241 0 nch w=1u l=180n
M616 t241 t237 0 0 nch w=1u l=180n
M617 t239 nw64 vdd vdd pch w=2u l=180n
M618 t239 t237 vdd vdd pch w=2u l=180n
CT242 t242 0 0.1f
M619 t239 nw64 t242 0 nch w=1u l=180n
M620 t242 t237 0 0 nch w=1u l=180n
M621 nw69 t238 vdd vdd pch w=2u l=180n
M622 nw69 t239 vdd vdd pch w=2u l=180n
CT243 t243 0 0.1f
M623 nw69 t238 t243 0 nch w=1u l=180n
M624 t243 t239 0 0 nch w=1u l=180n
Cnw69 nw69 0 2f
CT244 t244 0 0.1f
CT245 t245 0 0.1f
CT246 t246 0 0.1f
M625 t244 na10 vdd vdd pch w=2u l=180n
M626 t244 nb10 vdd vdd pch w=2u l=180n
CT247 t247 0 0.1f
M627 t244 na10 t247 0 nch w=1u l=180n
M628 t247 nb10 0 0 nch w=1u l=180n
M629 t245 na10 vdd vdd pch w=2u l=180n
M630 t245 t244 vdd vdd pch w=2u l=180n
CT248 t248 0 0.1f
M631 t245 na10 t248 0 nch w=1u l=180n
M632 t248 t244 0 0 nch w=1u l=180n
M633 t246 nb10 vdd vdd pch w=2u l=180n
M634 t246 t244 vdd vdd pch w=2u l=180n
CT249 t249 0 0.1f
M635 t246 nb10 t249 0 nch w=1u l=180n
M636 t249 t244 0 0 nch w=1u l=180n
M637 nw70 t245 vdd vdd pch w=2u l=180n
M638 nw70 t246 vdd vdd pch w=2u l=180n
CT250 t250 0 0.1f
M639 nw70 t245 t250 0 nch w=1u l=180n
M640 t250 t246 0 0 nch w=1u l=180n
Cnw70 nw70 0 2f
CT251 t251 0 0.1f
CT252 t252 0 0.1f
CT253 t253 0 0.1f
M641 t251 nw70 vdd vdd pch w=2u l=180n
M642 t251 nw67 vdd vdd pch w=2u l=180n
CT254 t254 0 0.1f
M643 t251 nw70 t254 0 nch w=1u l=180n
M644 t254 nw67 0 0 nch w=1u l=180n
M645 t252 nw70 vdd vdd pch w=2u l=180n
M646 t252 t251 vdd vdd pch w=2u l=180n
CT255 t255 0 0.1f
M647 t252 nw70 t255 0 nch w=1u l=180n
M648 t255 t251 0 0 nch w=1u l=180n
M649 t253 nw67 vdd vdd pch w=2u l=180n
M650 t253 t251 vdd vdd pch w=2u l=180n
CT256 t256 0 0.1f
M651 t253 nw67 t256 0 nch w=1u l=180n
M652 t256 t251 0 0 nch w=1u l=180n
M653 nw71 t252 vdd vdd pch w=2u l=180n
M654 nw71 t253 vdd vdd pch w=2u l=180n
CT257 t257 0 0.1f
M655 nw71 t252 t257 0 nch w=1u l=180n
M656 t257 t253 0 0 nch w=1u l=180n
Cnw71 nw71 0 2f
M657 nw72 na10 vdd vdd pch w=2u l=180n
M658 nw72 nb10 vdd vdd pch w=2u l=180n
CT258 t258 0 0.1f
M659 nw72 na10 t258 0 nch w=1u l=180n
M660 t258 nb10 0 0 nch w=1u l=180n
Cnw72 nw72 0 2f
M661 nw73 nw70 vdd vdd pch w=2u l=180n
M662 nw73 nw67 vdd vdd pch w=2u l=180n
CT259 t259 0 0.1f
M663 nw73 nw70 t259 0 nch w=1u l=180n
M664 t259 nw67 0 0 nch w=1u l=180n
Cnw73 nw73 0 2f
M665 nw74 nw72 vdd vdd pch w=2u l=180n
M666 nw74 nw73 vdd vdd pch w=2u l=180n
CT260 t260 0 0.1f
M667 nw74 nw72 t260 0 nch w=1u l=180n
M668 t260 nw73 0 0 nch w=1u l=180n
Cnw74 nw74 0 2f
CT261 t261 0 0.1f
M669 t261 nw71 vdd vdd pch w=2u l=180n
M670 t261 nw71 0 0 nch w=1u l=180n
M671 ns10 t261 vdd vdd pch w=2u l=180n
M672 ns10 t261 0 0 nch w=1u l=180n
Cns10 ns10 0 2f
CT262 t262 0 0.1f
CT263 t263 0 0.1f
CT264 t264 0 0.1f
M673 t262 nw69 vdd vdd pch w=2u l=180n
M674 t262 nw71 vdd vdd pch w=2u l=180n
CT265 t265 0 0.1f
M675 t262 nw69 t265 0 nch w=1u l=180n
M676 t265 nw71 0 0 nch w=1u l=180n
M677 t263 nw69 vdd vdd pch w=2u l=180n
M678 t263 t262 vdd vdd pch w=2u l=180n
CT266 t266 0 0.1f
M679 t263 nw69 t266 0 nch w=1u l=180n
M680 t266 t262 0 0 nch w=1u l=180n
M681 t264 nw71 vdd vdd pch w=2u l=180n
M682 t264 t262 vdd vdd pch w=2u l=180n
CT267 t267 0 0.1f
M683 t264 nw71 t267 0 nch w=1u l=180n
M684 t267 t262 0 0 nch w=1u l=180n
M685 nw76 t263 vdd vdd pch w=2u l=180n
M686 nw76 t264 vdd vdd pch w=2u l=180n
CT268 t268 0 0.1f
M687 nw76 t263 t268 0 nch w=1u l=180n
M688 t268 t264 0 0 nch w=1u l=180n
Cnw76 nw76 0 2f
CT269 t269 0 0.1f
CT270 t270 0 0.1f
CT271 t271 0 0.1f
M689 t269 na11 vdd vdd pch w=2u l=180n
M690 t269 nb11 vdd vdd pch w=2u l=180n
CT272 t272 0 0.1f
M691 t269 na11 t272 0 nch w=1u l=180n
M692 t272 nb11 0 0 nch w=1u l=180n
M693 t270 na11 vdd vdd pch w=2u l=180n
M694 t270 t269 vdd vdd pch w=2u l=180n
CT273 t273 0 0.1f
M695 t270 na11 t273 0 nch w=1u l=180n
M696 t273 t269 0 0 nch w=1u l=180n
M697 t271 nb11 vdd vdd pch w=2u l=180n
M698 t271 t269 vdd vdd pch w=2u l=180n
CT274 t274 0 0.1f
M699 t271 nb11 t274 0 nch w=1u l=180n
M700 t274 t269 0 0 nch w=1u l=180n
M701 nw77 t270 vdd vdd pch w=2u l=180n
M702 nw77 t271 vdd vdd pch w=2u l=180n
CT275 t275 0 0.1f
M703 nw77 t270 t275 0 nch w=1u l=180n
M704 t275 t271 0 0 nch w=1u l=180n
Cnw77 nw77 0 2f
CT276 t276 0 0.1f
CT277 t277 0 0.1f
CT278 t278 0 0.1f
M705 t276 nw77 vdd vdd pch w=2u l=180n
M706 t276 nw74 vdd vdd pch w=2u l=180n
CT279 t279 0 0.1f
M707 t276 nw77 t279 0 nch w=1u l=180n
M708 t279 nw74 0 0 nch w=1u l=180n
M709 t277 nw77 vdd vdd pch w=2u l=180n
M710 t277 t276 vdd vdd pch w=2u l=180n
CT280 t280 0 0.1f
M711 t277 nw77 t280 0 nch w=1u l=180n
M712 t280 t276 0 0 nch w=1u l=180n
M713 t278 nw74 vdd vdd pch w=2u l=180n
M714 t278 t276 vdd vdd pch w=2u l=180n
CT281 t281 0 0.1f
M715 t278 nw74 t281 0 nch w=1u l=180n
M716 t281 t276 0 0 nch w=1u l=180n
M717 nw78 t277 vdd vdd pch w=2u l=180n
M718 nw78 t278 vdd vdd pch w=2u l=180n
CT282 t282 0 0.1f
M719 nw78 t277 t282 0 nch w=1u l=180n
M720 t282 t278 0 0 nch w=1u l=180n
Cnw78 nw78 0 2f
M721 nw79 na11 vdd vdd pch w=2u l=180n
M722 nw79 nb11 vdd vdd pch w=2u l=180n
CT283 t283 0 0.1f
M723 nw79 na11 t283 0 nch w=1u l=180n
M724 t283 nb11 0 0 nch w=1u l=180n
Cnw79 nw79 0 2f
M725 nw80 nw77 vdd vdd pch w=2u l=180n
M726 nw80 nw74 vdd vdd pch w=2u l=180n
CT284 t284 0 0.1f
M727 nw80 nw77 t284 0 nch w=1u l=180n
M728 t284 nw74 0 0 nch w=1u l=180n
Cnw80 nw80 0 2f
M729 nw81 nw79 vdd vdd pch w=2u l=180n
M730 nw81 nw80 vdd vdd pch w=2u l=180n
CT285 t285 0 0.1f
M731 nw81 nw79 t285 0 nch w=1u l=180n
M732 t285 nw80 0 0 nch w=1u l=180n
Cnw81 nw81 0 2f
CT286 t286 0 0.1f
M733 t286 nw78 vdd vdd pch w=2u l=180n
M734 t286 nw78 0 0 nch w=1u l=180n
M735 ns11 t286 vdd vdd pch w=2u l=180n
M736 ns11 t286 0 0 nch w=1u l=180n
Cns11 ns11 0 2f
CT287 t287 0 0.1f
CT288 t288 0 0.1f
CT289 t289 0 0.1f
M737 t287 nw76 vdd vdd pch w=2u l=180n
M738 t287 nw78 vdd vdd pch w=2u l=180n
CT290 t290 0 0.1f
M739 t287 nw76 t290 0 nch w=1u l=180n
M740 t290 nw78 0 0 nch w=1u l=180n
M741 t288 nw76 vdd vdd pch w=2u l=180n
M742 t288 t287 vdd vdd pch w=2u l=180n
CT291 t291 0 0.1f
M743 t288 nw76 t291 0 nch w=1u l=180n
M744 t291 t287 0 0 nch w=1u l=180n
M745 t289 nw78 vdd vdd pch w=2u l=180n
M746 t289 t287 vdd vdd pch w=2u l=180n
CT292 t292 0 0.1f
M747 t289 nw78 t292 0 nch w=1u l=180n
M748 t292 t287 0 0 nch w=1u l=180n
M749 nw83 t288 vdd vdd pch w=2u l=180n
M750 nw83 t289 vdd vdd pch w=2u l=180n
CT293 t293 0 0.1f
M751 nw83 t288 t293 0 nch w=1u l=180n
M752 t293 t289 0 0 nch w=1u l=180n
Cnw83 nw83 0 2f
CT294 t294 0 0.1f
CT295 t295 0 0.1f
CT296 t296 0 0.1f
M753 t294 na12 vdd vdd pch w=2u l=180n
M754 t294 nb12 vdd vdd pch w=2u l=180n
CT297 t297 0 0.1f
M755 t294 na12 t297 0 nch w=1u l=180n
M756 t297 nb12 0 0 nch w=1u l=180n
M757 t295 na12 vdd vdd pch w=2u l=180n
M758 t295 t294 vdd vdd pch w=2u l=180n
CT298 t298 0 0.1f
M759 t295 na12 t298 0 nch w=1u l=180n
M760 t298 t294 0 0 nch w=1u l=180n
M761 t296 nb12 vdd vdd pch w=2u l=180n
M762 t296 t294 vdd vdd pch w=2u l=180n
CT299 t299 0 0.1f
M763 t296 nb12 t299 0 nch w=1u l=180n
M764 t299 t294 0 0 nch w=1u l=180n
M765 nw84 t295 vdd vdd pch w=2u l=180n
M766 nw84 t296 vdd vdd pch w=2u l=180n
CT300 t300 0 0.1f
M767 nw84 t295 t300 0 nch w=1u l=180n
M768 t300 t296 0 0 nch w=1u l=180n
Cnw84 nw84 0 2f
CT301 t301 0 0.1f
CT302 t302 0 0.1f
CT303 t303 0 0.1f
M769 t301 nw84 vdd vdd pch w=2u l=180n
M770 t301 nw81 vdd vdd pch w=2u l=180n
CT304 t304 0 0.1f
M771 t301 nw84 t304 0 nch w=1u l=180n
M772 t304 nw81 0 0 nch w=1u l=180n
M773 t302 nw84 vdd vdd pch w=2u l=180n
M774 t302 t301 vdd vdd pch w=2u l=180n
CT305 t305 0 0.1f
M775 t302 nw84 t305 0 nch w=1u l=180n
M776 t305 t301 0 0 nch w=1u l=180n
M777 t303 nw81 vdd vdd pch w=2u l=180n
M778 t303 t301 vdd vdd pch w=2u l=180n
CT306 t306 0 0.1f
M779 t303 nw81 t306 0 nch w=1u l=180n
M780 t306 t301 0 0 nch w=1u l=180n
M781 nw85 t302 vdd vdd pch w=2u l=180n
M782 nw85 t303 vdd vdd pch w=2u l=180n
CT307 t307 0 0.1f
M783 nw85 t302 t307 0 nch w=1u l=180n
M784 t307 t303 0 0 nch w=1u l=180n
Cnw85 nw85 0 2f
M785 nw86 na12 vdd vdd pch w=2u l=180n
M786 nw86 nb12 vdd vdd pch w=2u l=180n
CT308 t308 0 0.1f
M787 nw86 na12 t308 0 nch w=1u l=180n
M788 t308 nb12 0 0 nch w=1u l=180n
Cnw86 nw86 0 2f
M789 nw87 nw84 vdd vdd pch w=2u l=180n
M790 nw87 nw81 vdd vdd pch w=2u l=180n
CT309 t309 0 0.1f
M791 nw87 nw84 t309 0 nch w=1u l=180n
M792 t309 nw81 0 0 nch w=1u l=180n
Cnw87 nw87 0 2f
M793 nw88 nw86 vdd vdd pch w=2u l=180n
M794 nw88 nw87 vdd vdd pch w=2u l=180n
CT310 t310 0 0.1f
M795 nw88 nw86 t310 0 nch w=1u l=180n
M796 t310 nw87 0 0 nch w=1u l=180n
Cnw88 nw88 0 2f
CT311 t311 0 0.1f
M797 t311 nw85 vdd vdd pch w=2u l=180n
M798 t311 nw85 0 0 nch w=1u l=180n
M799 ns12 t311 vdd vdd pch w=2u l=180n
M800 ns12 t311 0 0 nch w=1u l=180n
Cns12 ns12 0 2f
CT312 t312 0 0.1f
CT313 t313 0 0.1f
CT314 t314 0 0.1f
M801 t312 nw83 vdd vdd pch w=2u l=180n
M802 t312 nw85 vdd vdd pch w=2u l=180n
CT315 t315 0 0.1f
M803 t312 nw83 t315 0 nch w=1u l=180n
M804 t315 nw85 0 0 nch w=1u l=180n
M805 t313 nw83 vdd vdd pch w=2u l=180n
M806 t313 t312 vdd vdd pch w=2u l=180n
CT316 t316 0 0.1f
M807 t313 nw83 t316 0 nch w=1u l=180n
M808 t316 t312 0 0 nch w=1u l=180n
M809 t314 nw85 vdd vdd pch w=2u l=180n
M810 t314 t312 vdd vdd pch w=2u l=180n
CT317 t317 0 0.1f
M811 t314 nw85 t317 0 nch w=1u l=180n
M812 t317 t312 0 0 nch w=1u l=180n
M813 nw90 t313 vdd vdd pch w=2u l=180n
M814 nw90 t314 vdd vdd pch w=2u l=180n
CT318 t318 0 0.1f
M815 nw90 t313 t318 0 nch w=1u l=180n
M816 t318 t314 0 0 nch w=1u l=180n
Cnw90 nw90 0 2f
CT319 t319 0 0.1f
CT320 t320 0 0.1f
CT321 t321 0 0.1f
M817 t319 na13 vdd vdd pch w=2u l=180n
M818 t319 nb13 vdd vdd pch w=2u l=180n
CT322 t322 0 0.1f
M819 t319 na13 t322 0 nch w=1u l=180n
M820 t322 nb13 0 0 nch w=1u l=180n
M821 t320 na13 vdd vdd pch w=2u l=180n
M822 t320 t319 vdd vdd pch w=2u l=180n
CT323 t323 0 0.1f
M823 t320 na13 t323 0 nch w=1u l=180n
M824 t323 t319 0 0 nch w=1u l=180n
M825 t321 nb13 vdd vdd pch w=2u l=180n
M826 t321 t319 vdd vdd pch w=2u l=180n
CT324 t324 0 0.1f
M827 t321 nb13 t324 0 nch w=1u l=180n
M828 t324 t319 0 0 nch w=1u l=180n
M829 nw91 t320 vdd vdd pch w=2u l=180n
M830 nw91 t321 vdd vdd pch w=2u l=180n
CT325 t325 0 0.1f
M831 nw91 t320 t325 0 nch w=1u l=180n
M832 t325 t321 0 0 nch w=1u l=180n
Cnw91 nw91 0 2f
CT326 t326 0 0.1f
CT327 t327 0 0.1f
CT328 t328 0 0.1f
M833 t326 nw91 vdd vdd pch w=2u l=180n
M834 t326 nw88 vdd vdd pch w=2u l=180n
CT329 t329 0 0.1f
M835 t326 nw91 t329 0 nch w=1u l=180n
M836 t329 nw88 0 0 nch w=1u l=180n
M837 t327 nw91 vdd vdd pch w=2u l=180n
M838 t327 t326 vdd vdd pch w=2u l=180n
CT330 t330 0 0.1f
M839 t327 nw91 t330 0 nch w=1u l=180n
M840 t330 t326 0 0 nch w=1u l=180n
M841 t328 nw88 vdd vdd pch w=2u l=180n
M842 t328 t326 vdd vdd pch w=2u l=180n
CT331 t331 0 0.1f
M843 t328 nw88 t331 0 nch w=1u l=180n
M844 t331 t326 0 0 nch w=1u l=180n
M845 nw92 t327 vdd vdd pch w=2u l=180n
M846 nw92 t328 vdd vdd pch w=2u l=180n
CT332 t332 0 0.1f
M847 nw92 t327 t332 0 nch w=1u l=180n
M848 t332 t328 0 0 nch w=1u l=180n
Cnw92 nw92 0 2f
M849 nw93 na13 vdd vdd pch w=2u l=180n
M850 nw93 nb13 vdd vdd pch w=2u l=180n
CT333 t333 0 0.1f
M851 nw93 na13 t333 0 nch w=1u l=180n
M852 t333 nb13 0 0 nch w=1u l=180n
Cnw93 nw93 0 2f
M853 nw94 nw91 vdd vdd pch w=2u l=180n
M854 nw94 nw88 vdd vdd pch w=2u l=180n
CT334 t334 0 0.1f
M855 nw94 nw91 t334 0 nch w=1u l=180n
M856 t334 nw88 0 0 nch w=1u l=180n
Cnw94 nw94 0 2f
M857 nw95 nw93 vdd vdd pch w=2u l=180n
M858 nw95 nw94 vdd vdd pch w=2u l=180n
CT335 t335 0 0.1f
M859 nw95 nw93 t335 0 nch w=1u l=180n
M860 t335 nw94 0 0 nch w=1u l=180n
Cnw95 nw95 0 2f
CT336 t336 0 0.1f
M861 t336 nw92 vdd vdd pch w=2u l=180n
M862 t336 nw92 0 0 nch w=1u l=180n
M863 ns13 t336 vdd vdd pch w=2u l=180n
M864 ns13 t336 0 0 nch w=1u l=180n
Cns13 ns13 0 2f
CT337 t337 0 0.1f
CT338 t338 0 0.1f
CT339 t339 0 0.1f
M865 t337 nw90 vdd vdd pch w=2u l=180n
M866 t337 nw92 vdd vdd pch w=2u l=180n
CT340 t340 0 0.1f
M867 t337 nw90 t340 0 nch w=1u l=180n
M868 t340 nw92 0 0 nch w=1u l=180n
M869 t338 nw90 vdd vdd pch w=2u l=180n
M870 t338 t337 vdd vdd pch w=2u l=180n
CT341 t341 0 0.1f
M871 t338 nw90 t341 0 nch w=1u l=180n
M872 t341 t337 0 0 nch w=1u l=180n
M873 t339 nw92 vdd vdd pch w=2u l=180n
M874 t339 t337 vdd vdd pch w=2u l=180n
CT342 t342 0 0.1f
M875 t339 nw92 t342 0 nch w=1u l=180n
M876 t342 t337 0 0 nch w=1u l=180n
M877 nw97 t338 vdd vdd pch w=2u l=180n
M878 nw97 t339 vdd vdd pch w=2u l=180n
CT343 t343 0 0.1f
M879 nw97 t338 t343 0 nch w=1u l=180n
M880 t343 t339 0 0 nch w=1u l=180n
Cnw97 nw97 0 2f
CT344 t344 0 0.1f
CT345 t345 0 0.1f
CT346 t346 0 0.1f
M881 t344 na14 vdd vdd pch w=2u l=180n
M882 t344 nb14 vdd vdd pch w=2u l=180n
CT347 t347 0 0.1f
M883 t344 na14 t347 0 nch w=1u l=180n
M884 t347 nb14 0 0 nch w=1u l=180n
M885 t345 na14 vdd vdd pch w=2u l=180n
M886 t345 t344 vdd vdd pch w=2u l=180n
CT348 t348 0 0.1f
M887 t345 na14 t348 0 nch w=1u l=180n
M888 t348 t344 0 0 nch w=1u l=180n
M889 t346 nb14 vdd vdd pch w=2u l=180n
M890 t346 t344 vdd vdd pch w=2u l=180n
CT349 t349 0 0.1f
M891 t346 nb14 t349 0 nch w=1u l=180n
M892 t349 t344 0 0 nch w=1u l=180n
M893 nw98 t345 vdd vdd pch w=2u l=180n
M894 nw98 t346 vdd vdd pch w=2u l=180n
CT350 t350 0 0.1f
M895 nw98 t345 t350 0 nch w=1u l=180n
M896 t350 t346 0 0 nch w=1u l=180n
Cnw98 nw98 0 2f
CT351 t351 0 0.1f
CT352 t352 0 0.1f
CT353 t353 0 0.1f
M897 t351 nw98 vdd vdd pch w=2u l=180n
M898 t351 nw95 vdd vdd pch w=2u l=180n
CT354 t354 0 0.1f
M899 t351 nw98 t354 0 nch w=1u l=180n
M900 t354 nw95 0 0 nch w=1u l=180n
M901 t352 nw98 vdd vdd pch w=2u l=180n
M902 t352 t351 vdd vdd pch w=2u l=180n
CT355 t355 0 0.1f
M903 t352 nw98 t355 0 nch w=1u l=180n
M904 t355 t351 0 0 nch w=1u l=180n
M905 t353 nw95 vdd vdd pch w=2u l=180n
M906 t353 t351 vdd vdd pch w=2u l=180n
CT356 t356 0 0.1f
M907 t353 nw95 t356 0 nch w=1u l=180n
M908 t356 t351 0 0 nch w=1u l=180n
M909 nw99 t352 vdd vdd pch w=2u l=180n
M910 nw99 t353 vdd vdd pch w=2u l=180n
CT357 t357 0 0.1f
M911 nw99 t352 t357 0 nch w=1u l=180n
M912 t357 t353 0 0 nch w=1u l=180n
Cnw99 nw99 0 2f
M913 nw100 na14 vdd vdd pch w=2u l=180n
M914 nw100 nb14 vdd vdd pch w=2u l=180n
CT358 t358 0 0.1f
M915 nw100 na14 t358 0 nch w=1u l=180n
M916 t358 nb14 0 0 nch w=1u l=180n
Cnw100 nw100 0 2f
M917 nw101 nw98 vdd vdd pch w=2u l=180n
M918 nw101 nw95 vdd vdd pch w=2u l=180n
CT359 t359 0 0.1f
M919 nw101 nw98 t359 0 nch w=1u l=180n
M920 t359 nw95 0 0 nch w=1u l=180n
Cnw101 nw101 0 2f
M921 nw102 nw100 vdd vdd pch w=2u l=180n
M922 nw102 nw101 vdd vdd pch w=2u l=180n
CT360 t360 0 0.1f
M923 nw102 nw100 t360 0 nch w=1u l=180n
M924 t360 nw101 0 0 nch w=1u l=180n
Cnw102 nw102 0 2f
CT361 t361 0 0.1f
M925 t361 nw99 vdd vdd pch w=2u l=180n
M926 t361 nw99 0 0 nch w=1u l=180n
M927 ns14 t361 vdd vdd pch w=2u l=180n
M928 ns14 t361 0 0 nch w=1u l=180n
Cns14 ns14 0 2f
CT362 t362 0 0.1f
CT363 t363 0 0.1f
CT364 t364 0 0.1f
M929 t362 nw97 vdd vdd pch w=2u l=180n
M930 t362 nw99 vdd vdd pch w=2u l=180n
CT365 t365 0 0.1f
M931 t362 nw97 t365 0 nch w=1u l=180n
M932 t365 nw99 0 0 nch w=1u l=180n
M933 t363 nw97 vdd vdd pch w=2u l=180n
M934 t363 t362 vdd vdd pch w=2u l=180n
CT366 t366 0 0.1f
M935 t363 nw97 t366 0 nch w=1u l=180n
M936 t366 t362 0 0 nch w=1u l=180n
M937 t364 nw99 vdd vdd pch w=2u l=180n
M938 t364 t362 vdd vdd pch w=2u l=180n
CT367 t367 0 0.1f
M939 t364 nw99 t367 0 nch w=1u l=180n
M940 t367 t362 0 0 nch w=1u l=180n
M941 nw104 t363 vdd vdd pch w=2u l=180n
M942 nw104 t364 vdd vdd pch w=2u l=180n
CT368 t368 0 0.1f
M943 nw104 t363 t368 0 nch w=1u l=180n
M944 t368 t364 0 0 nch w=1u l=180n
Cnw104 nw104 0 2f
CT369 t369 0 0.1f
CT370 t370 0 0.1f
CT371 t371 0 0.1f
M945 t369 na15 vdd vdd pch w=2u l=180n
M946 t369 nb15 vdd vdd pch w=2u l=180n
CT372 t372 0 0.1f
M947 t369 na15 t372 0 nch w=1u l=180n
M948 t372 nb15 0 0 nch w=1u l=180n
M949 t370 na15 vdd vdd pch w=2u l=180n
M950 t370 t369 vdd vdd pch w=2u l=180n
CT373 t373 0 0.1f
M951 t370 na15 t373 0 nch w=1u l=180n
M952 t373 t369 0 0 nch w=1u l=180n
M953 t371 nb15 vdd vdd pch w=2u l=180n
M954 t371 t369 vdd vdd pch w=2u l=180n
CT374 t374 0 0.1f
M955 t371 nb15 t374 0 nch w=1u l=180n
M956 t374 t369 0 0 nch w=1u l=180n
M957 nw105 t370 vdd vdd pch w=2u l=180n
M958 nw105 t371 vdd vdd pch w=2u l=180n
CT375 t375 0 0.1f
M959 nw105 t370 t375 0 nch w=1u l=180n
M960 t375 t371 0 0 nch w=1u l=180n
Cnw105 nw105 0 2f
CT376 t376 0 0.1f
CT377 t377 0 0.1f
CT378 t378 0 0.1f
M961 t376 nw105 vdd vdd pch w=2u l=180n
M962 t376 nw102 vdd vdd pch w=2u l=180n
CT379 t379 0 0.1f
M963 t376 nw105 t379 0 nch w=1u l=180n
M964 t379 nw102 0 0 nch w=1u l=180n
M965 t377 nw105 vdd vdd pch w=2u l=180n
M966 t377 t376 vdd vdd pch w=2u l=180n
CT380 t380 0 0.1f
M967 t377 nw105 t380 0 nch w=1u l=180n
M968 t380 t376 0 0 nch w=1u l=180n
M969 t378 nw102 vdd vdd pch w=2u l=180n
M970 t378 t376 vdd vdd pch w=2u l=180n
CT381 t381 0 0.1f
M971 t378 nw102 t381 0 nch w=1u l=180n
M972 t381 t376 0 0 nch w=1u l=180n
M973 nw106 t377 vdd vdd pch w=2u l=180n
M974 nw106 t378 vdd vdd pch w=2u l=180n
CT382 t382 0 0.1f
M975 nw106 t377 t382 0 nch w=1u l=180n
M976 t382 t378 0 0 nch w=1u l=180n
Cnw106 nw106 0 2f
M977 nw107 na15 vdd vdd pch w=2u l=180n
M978 nw107 nb15 vdd vdd pch w=2u l=180n
CT383 t383 0 0.1f
M979 nw107 na15 t383 0 nch w=1u l=180n
M980 t383 nb15 0 0 nch w=1u l=180n
Cnw107 nw107 0 2f
M981 nw108 nw105 vdd vdd pch w=2u l=180n
M982 nw108 nw102 vdd vdd pch w=2u l=180n
CT384 t384 0 0.1f
M983 nw108 nw105 t384 0 nch w=1u l=180n
M984 t384 nw102 0 0 nch w=1u l=180n
Cnw108 nw108 0 2f
M985 nw109 nw107 vdd vdd pch w=2u l=180n
M986 nw109 nw108 vdd vdd pch w=2u l=180n
CT385 t385 0 0.1f
M987 nw109 nw107 t385 0 nch w=1u l=180n
M988 t385 nw108 0 0 nch w=1u l=180n
Cnw109 nw109 0 2f
CT386 t386 0 0.1f
M989 t386 nw106 vdd vdd pch w=2u l=180n
M990 t386 nw106 0 0 nch w=1u l=180n
M991 ns15 t386 vdd vdd pch w=2u l=180n
M992 ns15 t386 0 0 nch w=1u l=180n
Cns15 ns15 0 2f
CT387 t387 0 0.1f
CT388 t388 0 0.1f
CT389 t389 0 0.1f
M993 t387 nw104 vdd vdd pch w=2u l=180n
M994 t387 nw106 vdd vdd pch w=2u l=180n
CT390 t390 0 0.1f
M995 t387 nw104 t390 0 nch w=1u l=180n
M996 t390 nw106 0 0 nch w=1u l=180n
M997 t388 nw104 vdd vdd pch w=2u l=180n
M998 t388 t387 vdd vdd pch w=2u l=180n
CT391 t391 0 0.1f
M999 t388 nw104 t391 0 nch w=1u l=180n
M1000 t391 t387 0 0 nch w=1u l=180n
M1001 t389 nw106 vdd vdd pch w=2u l=180n
M1002 t389 t387 vdd vdd pch w=2u l=180n
CT392 t392 0 0.1f
M1003 t389 nw106 t392 0 nch w=1u l=180n
M1004 t392 t387 0 0 nch w=1u l=180n
M1005 nw111 t388 vdd vdd pch w=2u l=180n
M1006 nw111 t389 vdd vdd pch w=2u l=180n
CT393 t393 0 0.1f
M1007 nw111 t388 t393 0 nch w=1u l=180n
M1008 t393 t389 0 0 nch w=1u l=180n
Cnw111 nw111 0 2f
CT394 t394 0 0.1f
CT395 t395 0 0.1f
CT396 t396 0 0.1f
M1009 t394 na16 vdd vdd pch w=2u l=180n
M1010 t394 nb16 vdd vdd pch w=2u l=180n
CT397 t397 0 0.1f
M1011 t394 na16 t397 0 nch w=1u l=180n
M1012 t397 nb16 0 0 nch w=1u l=180n
M1013 t395 na16 vdd vdd pch w=2u l=180n
M1014 t395 t394 vdd vdd pch w=2u l=180n
CT398 t398 0 0.1f
M1015 t395 na16 t398 0 nch w=1u l=180n
M1016 t398 t394 0 0 nch w=1u l=180n
M1017 t396 nb16 vdd vdd pch w=2u l=180n
M1018 t396 t394 vdd vdd pch w=2u l=180n
CT399 t399 0 0.1f
M1019 t396 nb16 t399 0 nch w=1u l=180n
M1020 t399 t394 0 0 nch w=1u l=180n
M1021 nw112 t395 vdd vdd pch w=2u l=180n
M1022 nw112 t396 vdd vdd pch w=2u l=180n
CT400 t400 0 0.1f
M1023 nw112 t395 t400 0 nch w=1u l=180n
M1024 t400 t396 0 0 nch w=1u l=180n
Cnw112 nw112 0 2f
CT401 t401 0 0.1f
CT402 t402 0 0.1f
CT403 t403 0 0.1f
M1025 t401 nw112 vdd vdd pch w=2u l=180n
M1026 t401 nw109 vdd vdd pch w=2u l=180n
CT404 t404 0 0.1f
M1027 t401 nw112 t404 0 nch w=1u l=180n
M1028 t404 nw109 0 0 nch w=1u l=180n
M1029 t402 nw112 vdd vdd pch w=2u l=180n
M1030 t402 t401 vdd vdd pch w=2u l=180n
CT405 t405 0 0.1f
M1031 t402 nw112 t405 0 nch w=1u l=180n
M1032 t405 t401 0 0 nch w=1u l=180n
M1033 t403 nw109 vdd vdd pch w=2u l=180n
M1034 t403 t401 vdd vdd pch w=2u l=180n
CT406 t406 0 0.1f
M1035 t403 nw109 t406 0 nch w=1u l=180n
M1036 t406 t401 0 0 nch w=1u l=180n
M1037 nw113 t402 vdd vdd pch w=2u l=180n
M1038 nw113 t403 vdd vdd pch w=2u l=180n
CT407 t407 0 0.1f
M1039 nw113 t402 t407 0 nch w=1u l=180n
M1040 t407 t403 0 0 nch w=1u l=180n
Cnw113 nw113 0 2f
M1041 nw114 na16 vdd vdd pch w=2u l=180n
M1042 nw114 nb16 vdd vdd pch w=2u l=180n
CT408 t408 0 0.1f
M1043 nw114 na16 t408 0 nch w=1u l=180n
M1044 t408 nb16 0 0 nch w=1u l=180n
Cnw114 nw114 0 2f
M1045 nw115 nw112 vdd vdd pch w=2u l=180n
M1046 nw115 nw109 vdd vdd pch w=2u l=180n
CT409 t409 0 0.1f
M1047 nw115 nw112 t409 0 nch w=1u l=180n
M1048 t409 nw109 0 0 nch w=1u l=180n
Cnw115 nw115 0 2f
M1049 nw116 nw114 vdd vdd pch w=2u l=180n
M1050 nw116 nw115 vdd vdd pch w=2u l=180n
CT410 t410 0 0.1f
M1051 nw116 nw114 t410 0 nch w=1u l=180n
M1052 t410 nw115 0 0 nch w=1u l=180n
Cnw116 nw116 0 2f
CT411 t411 0 0.1f
M1053 t411 nw113 vdd vdd pch w=2u l=180n
M1054 t411 nw113 0 0 nch w=1u l=180n
M1055 ns16 t411 vdd vdd pch w=2u l=180n
M1056 ns16 t411 0 0 nch w=1u l=180n
Cns16 ns16 0 2f
CT412 t412 0 0.1f
CT413 t413 0 0.1f
CT414 t414 0 0.1f
M1057 t412 nw111 vdd vdd pch w=2u l=180n
M1058 t412 nw113 vdd vdd pch w=2u l=180n
CT415 t415 0 0.1f
M1059 t412 nw111 t415 0 nch w=1u l=180n
M1060 t415 nw113 0 0 nch w=1u l=180n
M1061 t413 nw111 vdd vdd pch w=2u l=180n
M1062 t413 t412 vdd vdd pch w=2u l=180n
CT416 t416 0 0.1f
M1063 t413 nw111 t416 0 nch w=1u l=180n
M1064 t416 t412 0 0 nch w=1u l=180n
M1065 t414 nw113 vdd vdd pch w=2u l=180n
M1066 t414 t412 vdd vdd pch w=2u l=180n
CT417 t417 0 0.1f
M1067 t414 nw113 t417 0 nch w=1u l=180n
M1068 t417 t412 0 0 nch w=1u l=180n
M1069 nw118 t413 vdd vdd pch w=2u l=180n
M1070 nw118 t414 vdd vdd pch w=2u l=180n
CT418 t418 0 0.1f
M1071 nw118 t413 t418 0 nch w=1u l=180n
M1072 t418 t414 0 0 nch w=1u l=180n
Cnw118 nw118 0 2f
CT419 t419 0 0.1f
CT420 t420 0 0.1f
CT421 t421 0 0.1f
M1073 t419 na17 vdd vdd pch w=2u l=180n
M1074 t419 nb17 vdd vdd pch w=2u l=180n
CT422 t422 0 0.1f
M1075 t419 na17 t422 0 nch w=1u l=180n
M1076 t422 nb17 0 0 nch w=1u l=180n
M1077 t420 na17 vdd vdd pch w=2u l=180n
M1078 t420 t419 vdd vdd pch w=2u l=180n
CT423 t423 0 0.1f
M1079 t420 na17 t423 0 nch w=1u l=180n
M1080 t423 t419 0 0 nch w=1u l=180n
M1081 t421 nb17 vdd vdd pch w=2u l=180n
M1082 t421 t419 vdd vdd pch w=2u l=180n
CT424 t424 0 0.1f
M1083 t421 nb17 t424 0 nch w=1u l=180n
M1084 t424 t419 0 0 nch w=1u l=180n
M1085 nw119 t420 vdd vdd pch w=2u l=180n
M1086 nw119 t421 vdd vdd pch w=2u l=180n
CT425 t425 0 0.1f
M1087 nw119 t420 t425 0 nch w=1u l=180n
M1088 t425 t421 0 0 nch w=1u l=180n
Cnw119 nw119 0 2f
CT426 t426 0 0.1f
CT427 t427 0 0.1f
CT428 t428 0 0.1f
M1089 t426 nw119 vdd vdd pch w=2u l=180n
M1090 t426 nw116 vdd vdd pch w=2u l=180n
CT429 t429 0 0.1f
M1091 t426 nw119 t429 0 nch w=1u l=180n
M1092 t429 nw116 0 0 nch w=1u l=180n
M1093 t427 nw119 vdd vdd pch w=2u l=180n
M1094 t427 t426 vdd vdd pch w=2u l=180n
CT430 t430 0 0.1f
M1095 t427 nw119 t430 0 nch w=1u l=180n
M1096 t430 t426 0 0 nch w=1u l=180n
M1097 t428 nw116 vdd vdd pch w=2u l=180n
M1098 t428 t426 vdd vdd pch w=2u l=180n
CT431 t431 0 0.1f
M1099 t428 nw116 t431 0 nch w=1u l=180n
M1100 t431 t426 0 0 nch w=1u l=180n
M1101 nw120 t427 vdd vdd pch w=2u l=180n
M1102 nw120 t428 vdd vdd pch w=2u l=180n
CT432 t432 0 0.1f
M1103 nw120 t427 t432 0 nch w=1u l=180n
M1104 t432 t428 0 0 nch w=1u l=180n
Cnw120 nw120 0 2f
M1105 nw121 na17 vdd vdd pch w=2u l=180n
M1106 nw121 nb17 vdd vdd pch w=2u l=180n
CT433 t433 0 0.1f
M1107 nw121 na17 t433 0 nch w=1u l=180n
M1108 t433 nb17 0 0 nch w=1u l=180n
Cnw121 nw121 0 2f
M1109 nw122 nw119 vdd vdd pch w=2u l=180n
M1110 nw122 nw116 vdd vdd pch w=2u l=180n
CT434 t434 0 0.1f
M1111 nw122 nw119 t434 0 nch w=1u l=180n
M1112 t434 nw116 0 0 nch w=1u l=180n
Cnw122 nw122 0 2f
M1113 nw123 nw121 vdd vdd pch w=2u l=180n
M1114 nw123 nw122 vdd vdd pch w=2u l=180n
CT435 t435 0 0.1f
M1115 nw123 nw121 t435 0 nch w=1u l=180n
M1116 t435 nw122 0 0 nch w=1u l=180n
Cnw123 nw123 0 2f
CT436 t436 0 0.1f
M1117 t436 nw120 vdd vdd pch w=2u l=180n
M1118 t436 nw120 0 0 nch w=1u l=180n
M1119 ns17 t436 vdd vdd pch w=2u l=180n
M1120 ns17 t436 0 0 nch w=1u l=180n
Cns17 ns17 0 2f
CT437 t437 0 0.1f
CT438 t438 0 0.1f
CT439 t439 0 0.1f
M1121 t437 nw118 vdd vdd pch w=2u l=180n
M1122 t437 nw120 vdd vdd pch w=2u l=180n
CT440 t440 0 0.1f
M1123 t437 nw118 t440 0 nch w=1u l=180n
M1124 t440 nw120 0 0 nch w=1u l=180n
M1125 t438 nw118 vdd vdd pch w=2u l=180n
M1126 t438 t437 vdd vdd pch w=2u l=180n
CT441 t441 0 0.1f
M1127 t438 nw118 t441 0 nch w=1u l=180n
M1128 t441 t437 0 0 nch w=1u l=180n
M1129 t439 nw120 vdd vdd pch w=2u l=180n
M1130 t439 t437 vdd vdd pch w=2u l=180n
CT442 t442 0 0.1f
M1131 t439 nw120 t442 0 nch w=1u l=180n
M1132 t442 t437 0 0 nch w=1u l=180n
M1133 nw125 t438 vdd vdd pch w=2u l=180n
M1134 nw125 t439 vdd vdd pch w=2u l=180n
CT443 t443 0 0.1f
M1135 nw125 t438 t443 0 nch w=1u l=180n
M1136 t443 t439 0 0 nch w=1u l=180n
Cnw125 nw125 0 2f
CT444 t444 0 0.1f
CT445 t445 0 0.1f
CT446 t446 0 0.1f
M1137 t444 na18 vdd vdd pch w=2u l=180n
M1138 t444 nb18 vdd vdd pch w=2u l=180n
CT447 t447 0 0.1f
M1139 t444 na18 t447 0 nch w=1u l=180n
M1140 t447 nb18 0 0 nch w=1u l=180n
M1141 t445 na18 vdd vdd pch w=2u l=180n
M1142 t445 t444 vdd vdd pch w=2u l=180n
CT448 t448 0 0.1f
M1143 t445 na18 t448 0 nch w=1u l=180n
M1144 t448 t444 0 0 nch w=1u l=180n
M1145 t446 nb18 vdd vdd pch w=2u l=180n
M1146 t446 t444 vdd vdd pch w=2u l=180n
CT449 t449 0 0.1f
M1147 t446 nb18 t449 0 nch w=1u l=180n
M1148 t449 t444 0 0 nch w=1u l=180n
M1149 nw126 t445 vdd vdd pch w=2u l=180n
M1150 nw126 t446 vdd vdd pch w=2u l=180n
CT450 t450 0 0.1f
M1151 nw126 t445 t450 0 nch w=1u l=180n
M1152 t450 t446 0 0 nch w=1u l=180n
Cnw126 nw126 0 2f
CT451 t451 0 0.1f
CT452 t452 0 0.1f
CT453 t453 0 0.1f
M1153 t451 nw126 vdd vdd pch w=2u l=180n
M1154 t451 nw123 vdd vdd pch w=2u l=180n
CT454 t454 0 0.1f
M1155 t451 nw126 t454 0 nch w=1u l=180n
M1156 t454 nw123 0 0 nch w=1u l=180n
M1157 t452 nw126 vdd vdd pch w=2u l=180n
M1158 t452 t451 vdd vdd pch w=2u l=180n
CT455 t455 0 0.1f
M1159 t452 nw126 t455 0 nch w=1u l=180n
M1160 t455 t451 0 0 nch w=1u l=180n
M1161 t453 nw123 vdd vdd pch w=2u l=180n
M1162 t453 t451 vdd vdd pch w=2u l=180n
CT456 t456 0 0.1f
M1163 t453 nw123 t456 0 nch w=1u l=180n
M1164 t456 t451 0 0 nch w=1u l=180n
M1165 nw127 t452 vdd vdd pch w=2u l=180n
M1166 nw127 t453 vdd vdd pch w=2u l=180n
CT457 t457 0 0.1f
M1167 nw127 t452 t457 0 nch w=1u l=180n
M1168 t457 t453 0 0 nch w=1u l=180n
Cnw127 nw127 0 2f
M1169 nw128 na18 vdd vdd pch w=2u l=180n
M1170 nw128 nb18 vdd vdd pch w=2u l=180n
CT458 t458 0 0.1f
M1171 nw128 na18 t458 0 nch w=1u l=180n
M1172 t458 nb18 0 0 nch w=1u l=180n
Cnw128 nw128 0 2f
M1173 nw129 nw126 vdd vdd pch w=2u l=180n
M1174 nw129 nw123 vdd vdd pch w=2u l=180n
CT459 t459 0 0.1f
M1175 nw129 nw126 t459 0 nch w=1u l=180n
M1176 t459 nw123 0 0 nch w=1u l=180n
Cnw129 nw129 0 2f
M1177 nw130 nw128 vdd vdd pch w=2u l=180n
M1178 nw130 nw129 vdd vdd pch w=2u l=180n
CT460 t460 0 0.1f
M1179 nw130 nw128 t460 0 nch w=1u l=180n
M1180 t460 nw129 0 0 nch w=1u l=180n
Cnw130 nw130 0 2f
CT461 t461 0 0.1f
M1181 t461 nw127 vdd vdd pch w=2u l=180n
M1182 t461 nw127 0 0 nch w=1u l=180n
M1183 ns18 t461 vdd vdd pch w=2u l=180n
M1184 ns18 t461 0 0 nch w=1u l=180n
Cns18 ns18 0 2f
CT462 t462 0 0.1f
CT463 t463 0 0.1f
CT464 t464 0 0.1f
M1185 t462 nw125 vdd vdd pch w=2u l=180n
M1186 t462 nw127 vdd vdd pch w=2u l=180n
CT465 t465 0 0.1f
M1187 t462 nw125 t465 0 nch w=1u l=180n
M1188 t465 nw127 0 0 nch w=1u l=180n
M1189 t463 nw125 vdd vdd pch w=2u l=180n
M1190 t463 t462 vdd vdd pch w=2u l=180n
CT466 t466 0 0.1f
M1191 t463 nw125 t466 0 nch w=1u l=180n
M1192 t466 t462 0 0 nch w=1u l=180n
M1193 t464 nw127 vdd vdd pch w=2u l=180n
M1194 t464 t462 vdd vdd pch w=2u l=180n
CT467 t467 0 0.1f
M1195 t464 nw127 t467 0 nch w=1u l=180n
M1196 t467 t462 0 0 nch w=1u l=180n
M1197 nw132 t463 vdd vdd pch w=2u l=180n
M1198 nw132 t464 vdd vdd pch w=2u l=180n
CT468 t468 0 0.1f
M1199 nw132 t463 t468 0 nch w=1u l=180n
M1200 t468 t464 0 0 nch w=1u l=180n
Cnw132 nw132 0 2f
CT469 t469 0 0.1f
CT470 t470 0 0.1f
CT471 t471 0 0.1f
M1201 t469 na19 vdd vdd pch w=2u l=180n
M1202 t469 nb19 vdd vdd pch w=2u l=180n
CT472 t472 0 0.1f
M1203 t469 na19 t472 0 nch w=1u l=180n
M1204 t472 nb19 0 0 nch w=1u l=180n
M1205 t470 na19 vdd vdd pch w=2u l=180n
M1206 t470 t469 vdd vdd pch w=2u l=180n
CT473 t473 0 0.1f
M1207 t470 na19 t473 0 nch w=1u l=180n
M1208 t473 t469 0 0 nch w=1u l=180n
M1209 t471 nb19 vdd vdd pch w=2u l=180n
M1210 t471 t469 vdd vdd pch w=2u l=180n
CT474 t474 0 0.1f
M1211 t471 nb19 t474 0 nch w=1u l=180n
M1212 t474 t469 0 0 nch w=1u l=180n
M1213 nw133 t470 vdd vdd pch w=2u l=180n
M1214 nw133 t471 vdd vdd pch w=2u l=180n
CT475 t475 0 0.1f
M1215 nw133 t470 t475 0 nch w=1u l=180n
M1216 t475 t471 0 0 nch w=1u l=180n
Cnw133 nw133 0 2f
CT476 t476 0 0.1f
CT477 t477 0 0.1f
CT478 t478 0 0.1f
M1217 t476 nw133 vdd vdd pch w=2u l=180n
M1218 t476 nw130 vdd vdd pch w=2u l=180n
CT479 t479 0 0.1f
M1219 t476 nw133 t479 0 nch w=1u l=180n
M1220 t479 nw130 0 0 nch w=1u l=180n
M1221 t477 nw133 vdd vdd pch w=2u l=180n
M1222 t477 t476 vdd vdd pch w=2u l=180n
CT480 t480 0 0.1f
M1223 t477 nw133 t480 0 nch w=1u l=180n
M1224 t480 t476 0 0 nch w=1u l=180n
M1225 t478 nw130 vdd vdd pch w=2u l=180n
M1226 t478 t476 vdd vdd pch w=2u l=180n
CT481 t481 0 0.1f
M1227 t478 nw130 t481 0 nch w=1u l=180n
M1228 t481 t476 0 0 nch w=1u l=180n
M1229 nw134 t477 vdd vdd pch w=2u l=180n
M1230 nw134 t478 vdd vdd pch w=2u l=180n
CT482 t482 0 0.1f
M1231 nw134 t477 t482 0 nch w=1u l=180n
M1232 t482 t478 0 0 nch w=1u l=180n
Cnw134 nw134 0 2f
M1233 nw135 na19 vdd vdd pch w=2u l=180n
M1234 nw135 nb19 vdd vdd pch w=2u l=180n
CT483 t483 0 0.1f
M1235 nw135 na19 t483 0 nch w=1u l=180n
M1236 t483 nb19 0 0 nch w=1u l=180n
Cnw135 nw135 0 2f
M1237 nw136 nw133 vdd vdd pch w=2u l=180n
M1238 nw136 nw130 vdd vdd pch w=2u l=180n
CT484 t484 0 0.1f
M1239 nw136 nw133 t484 0 nch w=1u l=180n
M1240 t484 nw130 0 0 nch w=1u l=180n
Cnw136 nw136 0 2f
M1241 nw137 nw135 vdd vdd pch w=2u l=180n
M1242 nw137 nw136 vdd vdd pch w=2u l=180n
CT485 t485 0 0.1f
M1243 nw137 nw135 t485 0 nch w=1u l=180n
M1244 t485 nw136 0 0 nch w=1u l=180n
Cnw137 nw137 0 2f
CT486 t486 0 0.1f
M1245 t486 nw134 vdd vdd pch w=2u l=180n
M1246 t486 nw134 0 0 nch w=1u l=180n
M1247 ns19 t486 vdd vdd pch w=2u l=180n
M1248 ns19 t486 0 0 nch w=1u l=180n
Cns19 ns19 0 2f
CT487 t487 0 0.1f
CT488 t488 0 0.1f
CT489 t489 0 0.1f
M1249 t487 nw132 vdd vdd pch w=2u l=180n
M1250 t487 nw134 vdd vdd pch w=2u l=180n
CT490 t490 0 0.1f
M1251 t487 nw132 t490 0 nch w=1u l=180n
M1252 t490 nw134 0 0 nch w=1u l=180n
M1253 t488 nw132 vdd vdd pch w=2u l=180n
M1254 t488 t487 vdd vdd pch w=2u l=180n
CT491 t491 0 0.1f
M1255 t488 nw132 t491 0 nch w=1u l=180n
M1256 t491 t487 0 0 nch w=1u l=180n
M1257 t489 nw134 vdd vdd pch w=2u l=180n
M1258 t489 t487 vdd vdd pch w=2u l=180n
CT492 t492 0 0.1f
M1259 t489 nw134 t492 0 nch w=1u l=180n
M1260 t492 t487 0 0 nch w=1u l=180n
M1261 nw139 t488 vdd vdd pch w=2u l=180n
M1262 nw139 t489 vdd vdd pch w=2u l=180n
CT493 t493 0 0.1f
M1263 nw139 t488 t493 0 nch w=1u l=180n
M1264 t493 t489 0 0 nch w=1u l=180n
Cnw139 nw139 0 2f
CT494 t494 0 0.1f
CT495 t495 0 0.1f
CT496 t496 0 0.1f
M1265 t494 na20 vdd vdd pch w=2u l=180n
M1266 t494 nb20 vdd vdd pch w=2u l=180n
CT497 t497 0 0.1f
M1267 t494 na20 t497 0 nch w=1u l=180n
M1268 t497 nb20 0 0 nch w=1u l=180n
M1269 t495 na20 vdd vdd pch w=2u l=180n
M1270 t495 t494 vdd vdd pch w=2u l=180n
CT498 t498 0 0.1f
M1271 t495 na20 t498 0 nch w=1u l=180n
M1272 t498 t494 0 0 nch w=1u l=180n
M1273 t496 nb20 vdd vdd pch w=2u l=180n
M1274 t496 t494 vdd vdd pch w=2u l=180n
CT499 t499 0 0.1f
M1275 t496 nb20 t499 0 nch w=1u l=180n
M1276 t499 t494 0 0 nch w=1u l=180n
M1277 nw140 t495 vdd vdd pch w=2u l=180n
M1278 nw140 t496 vdd vdd pch w=2u l=180n
CT500 t500 0 0.1f
M1279 nw140 t495 t500 0 nch w=1u l=180n
M1280 t500 t496 0 0 nch w=1u l=180n
Cnw140 nw140 0 2f
CT501 t501 0 0.1f
CT502 t502 0 0.1f
CT503 t503 0 0.1f
M1281 t501 nw140 vdd vdd pch w=2u l=180n
M1282 t501 nw137 vdd vdd pch w=2u l=180n
CT504 t504 0 0.1f
M1283 t501 nw140 t504 0 nch w=1u l=180n
M1284 t504 nw137 0 0 nch w=1u l=180n
M1285 t502 nw140 vdd vdd pch w=2u l=180n
M1286 t502 t501 vdd vdd pch w=2u l=180n
CT505 t505 0 0.1f
M1287 t502 nw140 t505 0 nch w=1u l=180n
M1288 t505 t501 0 0 nch w=1u l=180n
M1289 t503 nw137 vdd vdd pch w=2u l=180n
M1290 t503 t501 vdd vdd pch w=2u l=180n
CT506 t506 0 0.1f
M1291 t503 nw137 t506 0 nch w=1u l=180n
M1292 t506 t501 0 0 nch w=1u l=180n
M1293 nw141 t502 vdd vdd pch w=2u l=180n
M1294 nw141 t503 vdd vdd pch w=2u l=180n
CT507 t507 0 0.1f
M1295 nw141 t502 t507 0 nch w=1u l=180n
M1296 t507 t503 0 0 nch w=1u l=180n
Cnw141 nw141 0 2f
M1297 nw142 na20 vdd vdd pch w=2u l=180n
M1298 nw142 nb20 vdd vdd pch w=2u l=180n
CT508 t508 0 0.1f
M1299 nw142 na20 t508 0 nch w=1u l=180n
M1300 t508 nb20 0 0 nch w=1u l=180n
Cnw142 nw142 0 2f
M1301 nw143 nw140 vdd vdd pch w=2u l=180n
M1302 nw143 nw137 vdd vdd pch w=2u l=180n
CT509 t509 0 0.1f
M1303 nw143 nw140 t509 0 nch w=1u l=180n
M1304 t509 nw137 0 0 nch w=1u l=180n
Cnw143 nw143 0 2f
M1305 nw144 nw142 vdd vdd pch w=2u l=180n
M1306 nw144 nw143 vdd vdd pch w=2u l=180n
CT510 t510 0 0.1f
M1307 nw144 nw142 t510 0 nch w=1u l=180n
M1308 t510 nw143 0 0 nch w=1u l=180n
Cnw144 nw144 0 2f
CT511 t511 0 0.1f
M1309 t511 nw141 vdd vdd pch w=2u l=180n
M1310 t511 nw141 0 0 nch w=1u l=180n
M1311 ns20 t511 vdd vdd pch w=2u l=180n
M1312 ns20 t511 0 0 nch w=1u l=180n
Cns20 ns20 0 2f
CT512 t512 0 0.1f
CT513 t513 0 0.1f
CT514 t514 0 0.1f
M1313 t512 nw139 vdd vdd pch w=2u l=180n
M1314 t512 nw141 vdd vdd pch w=2u l=180n
CT515 t515 0 0.1f
M1315 t512 nw139 t515 0 nch w=1u l=180n
M1316 t515 nw141 0 0 nch w=1u l=180n
M1317 t513 nw139 vdd vdd pch w=2u l=180n
M1318 t513 t512 vdd vdd pch w=2u l=180n
CT516 t516 0 0.1f
M1319 t513 nw139 t516 0 nch w=1u l=180n
M1320 t516 t512 0 0 nch w=1u l=180n
M1321 t514 nw141 vdd vdd pch w=2u l=180n
M1322 t514 t512 vdd vdd pch w=2u l=180n
CT517 t517 0 0.1f
M1323 t514 nw141 t517 0 nch w=1u l=180n
M1324 t517 t512 0 0 nch w=1u l=180n
M1325 nw146 t513 vdd vdd pch w=2u l=180n
M1326 nw146 t514 vdd vdd pch w=2u l=180n
CT518 t518 0 0.1f
M1327 nw146 t513 t518 0 nch w=1u l=180n
M1328 t518 t514 0 0 nch w=1u l=180n
Cnw146 nw146 0 2f
CT519 t519 0 0.1f
CT520 t520 0 0.1f
CT521 t521 0 0.1f
M1329 t519 na21 vdd vdd pch w=2u l=180n
M1330 t519 nb21 vdd vdd pch w=2u l=180n
CT522 t522 0 0.1f
M1331 t519 na21 t522 0 nch w=1u l=180n
M1332 t522 nb21 0 0 nch w=1u l=180n
M1333 t520 na21 vdd vdd pch w=2u l=180n
M1334 t520 t519 vdd vdd pch w=2u l=180n
CT523 t523 0 0.1f
M1335 t520 na21 t523 0 nch w=1u l=180n
M1336 t523 t519 0 0 nch w=1u l=180n
M1337 t521 nb21 vdd vdd pch w=2u l=180n
M1338 t521 t519 vdd vdd pch w=2u l=180n
CT524 t524 0 0.1f
M1339 t521 nb21 t524 0 nch w=1u l=180n
M1340 t524 t519 0 0 nch w=1u l=180n
M1341 nw147 t520 vdd vdd pch w=2u l=180n
M1342 nw147 t521 vdd vdd pch w=2u l=180n
CT525 t525 0 0.1f
M1343 nw147 t520 t525 0 nch w=1u l=180n
M1344 t525 t521 0 0 nch w=1u l=180n
Cnw147 nw147 0 2f
CT526 t526 0 0.1f
CT527 t527 0 0.1f
CT528 t528 0 0.1f
M1345 t526 nw147 vdd vdd pch w=2u l=180n
M1346 t526 nw144 vdd vdd pch w=2u l=180n
CT529 t529 0 0.1f
M1347 t526 nw147 t529 0 nch w=1u l=180n
M1348 t529 nw144 0 0 nch w=1u l=180n
M1349 t527 nw147 vdd vdd pch w=2u l=180n
M1350 t527 t526 vdd vdd pch w=2u l=180n
CT530 t530 0 0.1f
M1351 t527 nw147 t530 0 nch w=1u l=180n
M1352 t530 t526 0 0 nch w=1u l=180n
M1353 t528 nw144 vdd vdd pch w=2u l=180n
M1354 t528 t526 vdd vdd pch w=2u l=180n
CT531 t531 0 0.1f
M1355 t528 nw144 t531 0 nch w=1u l=180n
M1356 t531 t526 0 0 nch w=1u l=180n
M1357 nw148 t527 vdd vdd pch w=2u l=180n
M1358 nw148 t528 vdd vdd pch w=2u l=180n
CT532 t532 0 0.1f
M1359 nw148 t527 t532 0 nch w=1u l=180n
M1360 t532 t528 0 0 nch w=1u l=180n
Cnw148 nw148 0 2f
M1361 nw149 na21 vdd vdd pch w=2u l=180n
M1362 nw149 nb21 vdd vdd pch w=2u l=180n
CT533 t533 0 0.1f
M1363 nw149 na21 t533 0 nch w=1u l=180n
M1364 t533 nb21 0 0 nch w=1u l=180n
Cnw149 nw149 0 2f
M1365 nw150 nw147 vdd vdd pch w=2u l=180n
M1366 nw150 nw144 vdd vdd pch w=2u l=180n
CT534 t534 0 0.1f
M1367 nw150 nw147 t534 0 nch w=1u l=180n
M1368 t534 nw144 0 0 nch w=1u l=180n
Cnw150 nw150 0 2f
M1369 nw151 nw149 vdd vdd pch w=2u l=180n
M1370 nw151 nw150 vdd vdd pch w=2u l=180n
CT535 t535 0 0.1f
M1371 nw151 nw149 t535 0 nch w=1u l=180n
M1372 t535 nw150 0 0 nch w=1u l=180n
Cnw151 nw151 0 2f
CT536 t536 0 0.1f
M1373 t536 nw148 vdd vdd pch w=2u l=180n
M1374 t536 nw148 0 0 nch w=1u l=180n
M1375 ns21 t536 vdd vdd pch w=2u l=180n
M1376 ns21 t536 0 0 nch w=1u l=180n
Cns21 ns21 0 2f
CT537 t537 0 0.1f
CT538 t538 0 0.1f
CT539 t539 0 0.1f
M1377 t537 nw146 vdd vdd pch w=2u l=180n
M1378 t537 nw148 vdd vdd pch w=2u l=180n
CT540 t540 0 0.1f
M1379 t537 nw146 t540 0 nch w=1u l=180n
M1380 t540 nw148 0 0 nch w=1u l=180n
M1381 t538 nw146 vdd vdd pch w=2u l=180n
M1382 t538 t537 vdd vdd pch w=2u l=180n
CT541 t541 0 0.1f
M1383 t538 nw146 t541 0 nch w=1u l=180n
M1384 t541 t537 0 0 nch w=1u l=180n
M1385 t539 nw148 vdd vdd pch w=2u l=180n
M1386 t539 t537 vdd vdd pch w=2u l=180n
CT542 t542 0 0.1f
M1387 t539 nw148 t542 0 nch w=1u l=180n
M1388 t542 t537 0 0 nch w=1u l=180n
M1389 nw153 t538 vdd vdd pch w=2u l=180n
M1390 nw153 t539 vdd vdd pch w=2u l=180n
CT543 t543 0 0.1f
M1391 nw153 t538 t543 0 nch w=1u l=180n
M1392 t543 t539 0 0 nch w=1u l=180n
Cnw153 nw153 0 2f
CT544 t544 0 0.1f
CT545 t545 0 0.1f
CT546 t546 0 0.1f
M1393 t544 na22 vdd vdd pch w=2u l=180n
M1394 t544 nb22 vdd vdd pch w=2u l=180n
CT547 t547 0 0.1f
M1395 t544 na22 t547 0 nch w=1u l=180n
M1396 t547 nb22 0 0 nch w=1u l=180n
M1397 t545 na22 vdd vdd pch w=2u l=180n
M1398 t545 t544 vdd vdd pch w=2u l=180n
CT548 t548 0 0.1f
M1399 t545 na22 t548 0 nch w=1u l=180n
M1400 t548 t544 0 0 nch w=1u l=180n
M1401 t546 nb22 vdd vdd pch w=2u l=180n
M1402 t546 t544 vdd vdd pch w=2u l=180n
CT549 t549 0 0.1f
M1403 t546 nb22 t549 0 nch w=1u l=180n
M1404 t549 t544 0 0 nch w=1u l=180n
M1405 nw154 t545 vdd vdd pch w=2u l=180n
M1406 nw154 t546 vdd vdd pch w=2u l=180n
CT550 t550 0 0.1f
M1407 nw154 t545 t550 0 nch w=1u l=180n
M1408 t550 t546 0 0 nch w=1u l=180n
Cnw154 nw154 0 2f
CT551 t551 0 0.1f
CT552 t552 0 0.1f
CT553 t553 0 0.1f
M1409 t551 nw154 vdd vdd pch w=2u l=180n
M1410 t551 nw151 vdd vdd pch w=2u l=180n
CT554 t554 0 0.1f
M1411 t551 nw154 t554 0 nch w=1u l=180n
M1412 t554 nw151 0 0 nch w=1u l=180n
M1413 t552 nw154 vdd vdd pch w=2u l=180n
M1414 t552 t551 vdd vdd pch w=2u l=180n
CT555 t555 0 0.1f
M1415 t552 nw154 t555 0 nch w=1u l=180n
M1416 t555 t551 0 0 nch w=1u l=180n
M1417 t553 nw151 vdd vdd pch w=2u l=180n
M1418 t553 t551 vdd vdd pch w=2u l=180n
CT556 t556 0 0.1f
M1419 t553 nw151 t556 0 nch w=1u l=180n
M1420 t556 t551 0 0 nch w=1u l=180n
M1421 nw155 t552 vdd vdd pch w=2u l=180n
M1422 nw155 t553 vdd vdd pch w=2u l=180n
CT557 t557 0 0.1f
M1423 nw155 t552 t557 0 nch w=1u l=180n
M1424 t557 t553 0 0 nch w=1u l=180n
Cnw155 nw155 0 2f
M1425 nw156 na22 vdd vdd pch w=2u l=180n
M1426 nw156 nb22 vdd vdd pch w=2u l=180n
CT558 t558 0 0.1f
M1427 nw156 na22 t558 0 nch w=1u l=180n
M1428 t558 nb22 0 0 nch w=1u l=180n
Cnw156 nw156 0 2f
M1429 nw157 nw154 vdd vdd pch w=2u l=180n
M1430 nw157 nw151 vdd vdd pch w=2u l=180n
CT559 t559 0 0.1f
M1431 nw157 nw154 t559 0 nch w=1u l=180n
M1432 t559 nw151 0 0 nch w=1u l=180n
Cnw157 nw157 0 2f
M1433 nw158 nw156 vdd vdd pch w=2u l=180n
M1434 nw158 nw157 vdd vdd pch w=2u l=180n
CT560 t560 0 0.1f
M1435 nw158 nw156 t560 0 nch w=1u l=180n
M1436 t560 nw157 0 0 nch w=1u l=180n
Cnw158 nw158 0 2f
CT561 t561 0 0.1f
M1437 t561 nw155 vdd vdd pch w=2u l=180n
M1438 t561 nw155 0 0 nch w=1u l=180n
M1439 ns22 t561 vdd vdd pch w=2u l=180n
M1440 ns22 t561 0 0 nch w=1u l=180n
Cns22 ns22 0 2f
CT562 t562 0 0.1f
CT563 t563 0 0.1f
CT564 t564 0 0.1f
M1441 t562 nw153 vdd vdd pch w=2u l=180n
M1442 t562 nw155 vdd vdd pch w=2u l=180n
CT565 t565 0 0.1f
M1443 t562 nw153 t565 0 nch w=1u l=180n
M1444 t565 nw155 0 0 nch w=1u l=180n
M1445 t563 nw153 vdd vdd pch w=2u l=180n
M1446 t563 t562 vdd vdd pch w=2u l=180n
CT566 t566 0 0.1f
M1447 t563 nw153 t566 0 nch w=1u l=180n
M1448 t566 t562 0 0 nch w=1u l=180n
M1449 t564 nw155 vdd vdd pch w=2u l=180n
M1450 t564 t562 vdd vdd pch w=2u l=180n
CT567 t567 0 0.1f
M1451 t564 nw155 t567 0 nch w=1u l=180n
M1452 t567 t562 0 0 nch w=1u l=180n
M1453 nw160 t563 vdd vdd pch w=2u l=180n
M1454 nw160 t564 vdd vdd pch w=2u l=180n
CT568 t568 0 0.1f
M1455 nw160 t563 t568 0 nch w=1u l=180n
M1456 t568 t564 0 0 nch w=1u l=180n
Cnw160 nw160 0 2f
CT569 t569 0 0.1f
CT570 t570 0 0.1f
CT571 t571 0 0.1f
M1457 t569 na23 vdd vdd pch w=2u l=180n
M1458 t569 nb23 vdd vdd pch w=2u l=180n
CT572 t572 0 0.1f
M1459 t569 na23 t572 0 nch w=1u l=180n
M1460 t572 nb23 0 0 nch w=1u l=180n
M1461 t570 na23 vdd vdd pch w=2u l=180n
M1462 t570 t569 vdd vdd pch w=2u l=180n
CT573 t573 0 0.1f
M1463 t570 na23 t573 0 nch w=1u l=180n
M1464 t573 t569 0 0 nch w=1u l=180n
M1465 t571 nb23 vdd vdd pch w=2u l=180n
M1466 t571 t569 vdd vdd pch w=2u l=180n
CT574 t574 0 0.1f
M1467 t571 nb23 t574 0 nch w=1u l=180n
M1468 t574 t569 0 0 nch w=1u l=180n
M1469 nw161 t570 vdd vdd pch w=2u l=180n
M1470 nw161 t571 vdd vdd pch w=2u l=180n
CT575 t575 0 0.1f
M1471 nw161 t570 t575 0 nch w=1u l=180n
M1472 t575 t571 0 0 nch w=1u l=180n
Cnw161 nw161 0 2f
CT576 t576 0 0.1f
CT577 t577 0 0.1f
CT578 t578 0 0.1f
M1473 t576 nw161 vdd vdd pch w=2u l=180n
M1474 t576 nw158 vdd vdd pch w=2u l=180n
CT579 t579 0 0.1f
M1475 t576 nw161 t579 0 nch w=1u l=180n
M1476 t579 nw158 0 0 nch w=1u l=180n
M1477 t577 nw161 vdd vdd pch w=2u l=180n
M1478 t577 t576 vdd vdd pch w=2u l=180n
CT580 t580 0 0.1f
M1479 t577 nw161 t580 0 nch w=1u l=180n
M1480 t580 t576 0 0 nch w=1u l=180n
M1481 t578 nw158 vdd vdd pch w=2u l=180n
M1482 t578 t576 vdd vdd pch w=2u l=180n
CT581 t581 0 0.1f
M1483 t578 nw158 t581 0 nch w=1u l=180n
M1484 t581 t576 0 0 nch w=1u l=180n
M1485 nw162 t577 vdd vdd pch w=2u l=180n
M1486 nw162 t578 vdd vdd pch w=2u l=180n
CT582 t582 0 0.1f
M1487 nw162 t577 t582 0 nch w=1u l=180n
M1488 t582 t578 0 0 nch w=1u l=180n
Cnw162 nw162 0 2f
M1489 nw163 na23 vdd vdd pch w=2u l=180n
M1490 nw163 nb23 vdd vdd pch w=2u l=180n
CT583 t583 0 0.1f
M1491 nw163 na23 t583 0 nch w=1u l=180n
M1492 t583 nb23 0 0 nch w=1u l=180n
Cnw163 nw163 0 2f
M1493 nw164 nw161 vdd vdd pch w=2u l=180n
M1494 nw164 nw158 vdd vdd pch w=2u l=180n
CT584 t584 0 0.1f
M1495 nw164 nw161 t584 0 nch w=1u l=180n
M1496 t584 nw158 0 0 nch w=1u l=180n
Cnw164 nw164 0 2f
M1497 nw165 nw163 vdd vdd pch w=2u l=180n
M1498 nw165 nw164 vdd vdd pch w=2u l=180n
CT585 t585 0 0.1f
M1499 nw165 nw163 t585 0 nch w=1u l=180n
M1500 t585 nw164 0 0 nch w=1u l=180n
Cnw165 nw165 0 2f
CT586 t586 0 0.1f
M1501 t586 nw162 vdd vdd pch w=2u l=180n
M1502 t586 nw162 0 0 nch w=1u l=180n
M1503 ns23 t586 vdd vdd pch w=2u l=180n
M1504 ns23 t586 0 0 nch w=1u l=180n
Cns23 ns23 0 2f
CT587 t587 0 0.1f
CT588 t588 0 0.1f
CT589 t589 0 0.1f
M1505 t587 nw160 vdd vdd pch w=2u l=180n
M1506 t587 nw162 vdd vdd pch w=2u l=180n
CT590 t590 0 0.1f
M1507 t587 nw160 t590 0 nch w=1u l=180n
M1508 t590 nw162 0 0 nch w=1u l=180n
M1509 t588 nw160 vdd vdd pch w=2u l=180n
M1510 t588 t587 vdd vdd pch w=2u l=180n
CT591 t591 0 0.1f
M1511 t588 nw160 t591 0 nch w=1u l=180n
M1512 t591 t587 0 0 nch w=1u l=180n
M1513 t589 nw162 vdd vdd pch w=2u l=180n
M1514 t589 t587 vdd vdd pch w=2u l=180n
CT592 t592 0 0.1f
M1515 t589 nw162 t592 0 nch w=1u l=180n
M1516 t592 t587 0 0 nch w=1u l=180n
M1517 nw167 t588 vdd vdd pch w=2u l=180n
M1518 nw167 t589 vdd vdd pch w=2u l=180n
CT593 t593 0 0.1f
M1519 nw167 t588 t593 0 nch w=1u l=180n
M1520 t593 t589 0 0 nch w=1u l=180n
Cnw167 nw167 0 2f
CT594 t594 0 0.1f
CT595 t595 0 0.1f
CT596 t596 0 0.1f
M1521 t594 na24 vdd vdd pch w=2u l=180n
M1522 t594 nb24 vdd vdd pch w=2u l=180n
CT597 t597 0 0.1f
M1523 t594 na24 t597 0 nch w=1u l=180n
M1524 t597 nb24 0 0 nch w=1u l=180n
M1525 t595 na24 vdd vdd pch w=2u l=180n
M1526 t595 t594 vdd vdd pch w=2u l=180n
CT598 t598 0 0.1f
M1527 t595 na24 t598 0 nch w=1u l=180n
M1528 t598 t594 0 0 nch w=1u l=180n
M1529 t596 nb24 vdd vdd pch w=2u l=180n
M1530 t596 t594 vdd vdd pch w=2u l=180n
CT599 t599 0 0.1f
M1531 t596 nb24 t599 0 nch w=1u l=180n
M1532 t599 t594 0 0 nch w=1u l=180n
M1533 nw168 t595 vdd vdd pch w=2u l=180n
M1534 nw168 t596 vdd vdd pch w=2u l=180n
CT600 t600 0 0.1f
M1535 nw168 t595 t600 0 nch w=1u l=180n
M1536 t600 t596 0 0 nch w=1u l=180n
Cnw168 nw168 0 2f
CT601 t601 0 0.1f
CT602 t602 0 0.1f
CT603 t603 0 0.1f
M1537 t601 nw168 vdd vdd pch w=2u l=180n
M1538 t601 nw165 vdd vdd pch w=2u l=180n
CT604 t604 0 0.1f
M1539 t601 nw168 t604 0 nch w=1u l=180n
M1540 t604 nw165 0 0 nch w=1u l=180n
M1541 t602 nw168 vdd vdd pch w=2u l=180n
M1542 t602 t601 vdd vdd pch w=2u l=180n
CT605 t605 0 0.1f
M1543 t602 nw168 t605 0 nch w=1u l=180n
M1544 t605 t601 0 0 nch w=1u l=180n
M1545 t603 nw165 vdd vdd pch w=2u l=180n
M1546 t603 t601 vdd vdd pch w=2u l=180n
CT606 t606 0 0.1f
M1547 t603 nw165 t606 0 nch w=1u l=180n
M1548 t606 t601 0 0 nch w=1u l=180n
M1549 nw169 t602 vdd vdd pch w=2u l=180n
M1550 nw169 t603 vdd vdd pch w=2u l=180n
CT607 t607 0 0.1f
M1551 nw169 t602 t607 0 nch w=1u l=180n
M1552 t607 t603 0 0 nch w=1u l=180n
Cnw169 nw169 0 2f
M1553 nw170 na24 vdd vdd pch w=2u l=180n
M1554 nw170 nb24 vdd vdd pch w=2u l=180n
CT608 t608 0 0.1f
M1555 nw170 na24 t608 0 nch w=1u l=180n
M1556 t608 nb24 0 0 nch w=1u l=180n
Cnw170 nw170 0 2f
M1557 nw171 nw168 vdd vdd pch w=2u l=180n
M1558 nw171 nw165 vdd vdd pch w=2u l=180n
CT609 t609 0 0.1f
M1559 nw171 nw168 t609 0 nch w=1u l=180n
M1560 t609 nw165 0 0 nch w=1u l=180n
Cnw171 nw171 0 2f
M1561 nw172 nw170 vdd vdd pch w=2u l=180n
M1562 nw172 nw171 vdd vdd pch w=2u l=180n
CT610 t610 0 0.1f
M1563 nw172 nw170 t610 0 nch w=1u l=180n
M1564 t610 nw171 0 0 nch w=1u l=180n
Cnw172 nw172 0 2f
CT611 t611 0 0.1f
M1565 t611 nw169 vdd vdd pch w=2u l=180n
M1566 t611 nw169 0 0 nch w=1u l=180n
M1567 ns24 t611 vdd vdd pch w=2u l=180n
M1568 ns24 t611 0 0 nch w=1u l=180n
Cns24 ns24 0 2f
CT612 t612 0 0.1f
CT613 t613 0 0.1f
CT614 t614 0 0.1f
M1569 t612 nw167 vdd vdd pch w=2u l=180n
M1570 t612 nw169 vdd vdd pch w=2u l=180n
CT615 t615 0 0.1f
M1571 t612 nw167 t615 0 nch w=1u l=180n
M1572 t615 nw169 0 0 nch w=1u l=180n
M1573 t613 nw167 vdd vdd pch w=2u l=180n
M1574 t613 t612 vdd vdd pch w=2u l=180n
CT616 t616 0 0.1f
M1575 t613 nw167 t616 0 nch w=1u l=180n
M1576 t616 t612 0 0 nch w=1u l=180n
M1577 t614 nw169 vdd vdd pch w=2u l=180n
M1578 t614 t612 vdd vdd pch w=2u l=180n
CT617 t617 0 0.1f
M1579 t614 nw169 t617 0 nch w=1u l=180n
M1580 t617 t612 0 0 nch w=1u l=180n
M1581 nw174 t613 vdd vdd pch w=2u l=180n
M1582 nw174 t614 vdd vdd pch w=2u l=180n
CT618 t618 0 0.1f
M1583 nw174 t613 t618 0 nch w=1u l=180n
M1584 t618 t614 0 0 nch w=1u l=180n
Cnw174 nw174 0 2f
CT619 t619 0 0.1f
CT620 t620 0 0.1f
CT621 t621 0 0.1f
M1585 t619 na25 vdd vdd pch w=2u l=180n
M1586 t619 nb25 vdd vdd pch w=2u l=180n
CT622 t622 0 0.1f
M1587 t619 na25 t622 0 nch w=1u l=180n
M1588 t622 nb25 0 0 nch w=1u l=180n
M1589 t620 na25 vdd vdd pch w=2u l=180n
M1590 t620 t619 vdd vdd pch w=2u l=180n
CT623 t623 0 0.1f
M1591 t620 na25 t623 0 nch w=1u l=180n
M1592 t623 t619 0 0 nch w=1u l=180n
M1593 t621 nb25 vdd vdd pch w=2u l=180n
M1594 t621 t619 vdd vdd pch w=2u l=180n
CT624 t624 0 0.1f
M1595 t621 nb25 t624 0 nch w=1u l=180n
M1596 t624 t619 0 0 nch w=1u l=180n
M1597 nw175 t620 vdd vdd pch w=2u l=180n
M1598 nw175 t621 vdd vdd pch w=2u l=180n
CT625 t625 0 0.1f
M1599 nw175 t620 t625 0 nch w=1u l=180n
M1600 t625 t621 0 0 nch w=1u l=180n
Cnw175 nw175 0 2f
CT626 t626 0 0.1f
CT627 t627 0 0.1f
CT628 t628 0 0.1f
M1601 t626 nw175 vdd vdd pch w=2u l=180n
M1602 t626 nw172 vdd vdd pch w=2u l=180n
CT629 t629 0 0.1f
M1603 t626 nw175 t629 0 nch w=1u l=180n
M1604 t629 nw172 0 0 nch w=1u l=180n
M1605 t627 nw175 vdd vdd pch w=2u l=180n
M1606 t627 t626 vdd vdd pch w=2u l=180n
CT630 t630 0 0.1f
M1607 t627 nw175 t630 0 nch w=1u l=180n
M1608 t630 t626 0 0 nch w=1u l=180n
M1609 t628 nw172 vdd vdd pch w=2u l=180n
M1610 t628 t626 vdd vdd pch w=2u l=180n
CT631 t631 0 0.1f
M1611 t628 nw172 t631 0 nch w=1u l=180n
M1612 t631 t626 0 0 nch w=1u l=180n
M1613 nw176 t627 vdd vdd pch w=2u l=180n
M1614 nw176 t628 vdd vdd pch w=2u l=180n
CT632 t632 0 0.1f
M1615 nw176 t627 t632 0 nch w=1u l=180n
M1616 t632 t628 0 0 nch w=1u l=180n
Cnw176 nw176 0 2f
M1617 nw177 na25 vdd vdd pch w=2u l=180n
M1618 nw177 nb25 vdd vdd pch w=2u l=180n
CT633 t633 0 0.1f
M1619 nw177 na25 t633 0 nch w=1u l=180n
M1620 t633 nb25 0 0 nch w=1u l=180n
Cnw177 nw177 0 2f
M1621 nw178 nw175 vdd vdd pch w=2u l=180n
M1622 nw178 nw172 vdd vdd pch w=2u l=180n
CT634 t634 0 0.1f
M1623 nw178 nw175 t634 0 nch w=1u l=180n
M1624 t634 nw172 0 0 nch w=1u l=180n
Cnw178 nw178 0 2f
M1625 nw179 nw177 vdd vdd pch w=2u l=180n
M1626 nw179 nw178 vdd vdd pch w=2u l=180n
CT635 t635 0 0.1f
M1627 nw179 nw177 t635 0 nch w=1u l=180n
M1628 t635 nw178 0 0 nch w=1u l=180n
Cnw179 nw179 0 2f
CT636 t636 0 0.1f
M1629 t636 nw176 vdd vdd pch w=2u l=180n
M1630 t636 nw176 0 0 nch w=1u l=180n
M1631 ns25 t636 vdd vdd pch w=2u l=180n
M1632 ns25 t636 0 0 nch w=1u l=180n
Cns25 ns25 0 2f
CT637 t637 0 0.1f
CT638 t638 0 0.1f
CT639 t639 0 0.1f
M1633 t637 nw174 vdd vdd pch w=2u l=180n
M1634 t637 nw176 vdd vdd pch w=2u l=180n
CT640 t640 0 0.1f
M1635 t637 nw174 t640 0 nch w=1u l=180n
M1636 t640 nw176 0 0 nch w=1u l=180n
M1637 t638 nw174 vdd vdd pch w=2u l=180n
M1638 t638 t637 vdd vdd pch w=2u l=180n
CT641 t641 0 0.1f
M1639 t638 nw174 t641 0 nch w=1u l=180n
M1640 t641 t637 0 0 nch w=1u l=180n
M1641 t639 nw176 vdd vdd pch w=2u l=180n
M1642 t639 t637 vdd vdd pch w=2u l=180n
CT642 t642 0 0.1f
M1643 t639 nw176 t642 0 nch w=1u l=180n
M1644 t642 t637 0 0 nch w=1u l=180n
M1645 nw181 t638 vdd vdd pch w=2u l=180n
M1646 nw181 t639 vdd vdd pch w=2u l=180n
CT643 t643 0 0.1f
M1647 nw181 t638 t643 0 nch w=1u l=180n
M1648 t643 t639 0 0 nch w=1u l=180n
Cnw181 nw181 0 2f
CT644 t644 0 0.1f
CT645 t645 0 0.1f
CT646 t646 0 0.1f
M1649 t644 na26 vdd vdd pch w=2u l=180n
M1650 t644 nb26 vdd vdd pch w=2u l=180n
CT647 t647 0 0.1f
M1651 t644 na26 t647 0 nch w=1u l=180n
M1652 t647 nb26 0 0 nch w=1u l=180n
M1653 t645 na26 vdd vdd pch w=2u l=180n
M1654 t645 t644 vdd vdd pch w=2u l=180n
CT648 t648 0 0.1f
M1655 t645 na26 t648 0 nch w=1u l=180n
M1656 t648 t644 0 0 nch w=1u l=180n
M1657 t646 nb26 vdd vdd pch w=2u l=180n
M1658 t646 t644 vdd vdd pch w=2u l=180n
CT649 t649 0 0.1f
M1659 t646 nb26 t649 0 nch w=1u l=180n
M1660 t649 t644 0 0 nch w=1u l=180n
M1661 nw182 t645 vdd vdd pch w=2u l=180n
M1662 nw182 t646 vdd vdd pch w=2u l=180n
CT650 t650 0 0.1f
M1663 nw182 t645 t650 0 nch w=1u l=180n
M1664 t650 t646 0 0 nch w=1u l=180n
Cnw182 nw182 0 2f
CT651 t651 0 0.1f
CT652 t652 0 0.1f
CT653 t653 0 0.1f
M1665 t651 nw182 vdd vdd pch w=2u l=180n
M1666 t651 nw179 vdd vdd pch w=2u l=180n
CT654 t654 0 0.1f
M1667 t651 nw182 t654 0 nch w=1u l=180n
M1668 t654 nw179 0 0 nch w=1u l=180n
M1669 t652 nw182 vdd vdd pch w=2u l=180n
M1670 t652 t651 vdd vdd pch w=2u l=180n
CT655 t655 0 0.1f
M1671 t652 nw182 t655 0 nch w=1u l=180n
M1672 t655 t651 0 0 nch w=1u l=180n
M1673 t653 nw179 vdd vdd pch w=2u l=180n
M1674 t653 t651 vdd vdd pch w=2u l=180n
CT656 t656 0 0.1f
M1675 t653 nw179 t656 0 nch w=1u l=180n
M1676 t656 t651 0 0 nch w=1u l=180n
M1677 nw183 t652 vdd vdd pch w=2u l=180n
M1678 nw183 t653 vdd vdd pch w=2u l=180n
CT657 t657 0 0.1f
M1679 nw183 t652 t657 0 nch w=1u l=180n
M1680 t657 t653 0 0 nch w=1u l=180n
Cnw183 nw183 0 2f
M1681 nw184 na26 vdd vdd pch w=2u l=180n
M1682 nw184 nb26 vdd vdd pch w=2u l=180n
CT658 t658 0 0.1f
M1683 nw184 na26 t658 0 nch w=1u l=180n
M1684 t658 nb26 0 0 nch w=1u l=180n
Cnw184 nw184 0 2f
M1685 nw185 nw182 vdd vdd pch w=2u l=180n
M1686 nw185 nw179 vdd vdd pch w=2u l=180n
CT659 t659 0 0.1f
M1687 nw185 nw182 t659 0 nch w=1u l=180n
M1688 t659 nw179 0 0 nch w=1u l=180n
Cnw185 nw185 0 2f
M1689 nw186 nw184 vdd vdd pch w=2u l=180n
M1690 nw186 nw185 vdd vdd pch w=2u l=180n
CT660 t660 0 0.1f
M1691 nw186 nw184 t660 0 nch w=1u l=180n
M1692 t660 nw185 0 0 nch w=1u l=180n
Cnw186 nw186 0 2f
CT661 t661 0 0.1f
M1693 t661 nw183 vdd vdd pch w=2u l=180n
M1694 t661 nw183 0 0 nch w=1u l=180n
M1695 ns26 t661 vdd vdd pch w=2u l=180n
M1696 ns26 t661 0 0 nch w=1u l=180n
Cns26 ns26 0 2f
CT662 t662 0 0.1f
CT663 t663 0 0.1f
CT664 t664 0 0.1f
M1697 t662 nw181 vdd vdd pch w=2u l=180n
M1698 t662 nw183 vdd vdd pch w=2u l=180n
CT665 t665 0 0.1f
M1699 t662 nw181 t665 0 nch w=1u l=180n
M1700 t665 nw183 0 0 nch w=1u l=180n
M1701 t663 nw181 vdd vdd pch w=2u l=180n
M1702 t663 t662 vdd vdd pch w=2u l=180n
CT666 t666 0 0.1f
M1703 t663 nw181 t666 0 nch w=1u l=180n
M1704 t666 t662 0 0 nch w=1u l=180n
M1705 t664 nw183 vdd vdd pch w=2u l=180n
M1706 t664 t662 vdd vdd pch w=2u l=180n
CT667 t667 0 0.1f
M1707 t664 nw183 t667 0 nch w=1u l=180n
M1708 t667 t662 0 0 nch w=1u l=180n
M1709 nw188 t663 vdd vdd pch w=2u l=180n
M1710 nw188 t664 vdd vdd pch w=2u l=180n
CT668 t668 0 0.1f
M1711 nw188 t663 t668 0 nch w=1u l=180n
M1712 t668 t664 0 0 nch w=1u l=180n
Cnw188 nw188 0 2f
CT669 t669 0 0.1f
CT670 t670 0 0.1f
CT671 t671 0 0.1f
M1713 t669 na27 vdd vdd pch w=2u l=180n
M1714 t669 nb27 vdd vdd pch w=2u l=180n
CT672 t672 0 0.1f
M1715 t669 na27 t672 0 nch w=1u l=180n
M1716 t672 nb27 0 0 nch w=1u l=180n
M1717 t670 na27 vdd vdd pch w=2u l=180n
M1718 t670 t669 vdd vdd pch w=2u l=180n
CT673 t673 0 0.1f
M1719 t670 na27 t673 0 nch w=1u l=180n
M1720 t673 t669 0 0 nch w=1u l=180n
M1721 t671 nb27 vdd vdd pch w=2u l=180n
M1722 t671 t669 vdd vdd pch w=2u l=180n
CT674 t674 0 0.1f
M1723 t671 nb27 t674 0 nch w=1u l=180n
M1724 t674 t669 0 0 nch w=1u l=180n
M1725 nw189 t670 vdd vdd pch w=2u l=180n
M1726 nw189 t671 vdd vdd pch w=2u l=180n
CT675 t675 0 0.1f
M1727 nw189 t670 t675 0 nch w=1u l=180n
M1728 t675 t671 0 0 nch w=1u l=180n
Cnw189 nw189 0 2f
CT676 t676 0 0.1f
CT677 t677 0 0.1f
CT678 t678 0 0.1f
M1729 t676 nw189 vdd vdd pch w=2u l=180n
M1730 t676 nw186 vdd vdd pch w=2u l=180n
CT679 t679 0 0.1f
M1731 t676 nw189 t679 0 nch w=1u l=180n
M1732 t679 nw186 0 0 nch w=1u l=180n
M1733 t677 nw189 vdd vdd pch w=2u l=180n
M1734 t677 t676 vdd vdd pch w=2u l=180n
CT680 t680 0 0.1f
M1735 t677 nw189 t680 0 nch w=1u l=180n
M1736 t680 t676 0 0 nch w=1u l=180n
M1737 t678 nw186 vdd vdd pch w=2u l=180n
M1738 t678 t676 vdd vdd pch w=2u l=180n
CT681 t681 0 0.1f
M1739 t678 nw186 t681 0 nch w=1u l=180n
M1740 t681 t676 0 0 nch w=1u l=180n
M1741 nw190 t677 vdd vdd pch w=2u l=180n
M1742 nw190 t678 vdd vdd pch w=2u l=180n
CT682 t682 0 0.1f
M1743 nw190 t677 t682 0 nch w=1u l=180n
M1744 t682 t678 0 0 nch w=1u l=180n
Cnw190 nw190 0 2f
M1745 nw191 na27 vdd vdd pch w=2u l=180n
M1746 nw191 nb27 vdd vdd pch w=2u l=180n
CT683 t683 0 0.1f
M1747 nw191 na27 t683 0 nch w=1u l=180n
M1748 t683 nb27 0 0 nch w=1u l=180n
Cnw191 nw191 0 2f
M1749 nw192 nw189 vdd vdd pch w=2u l=180n
M1750 nw192 nw186 vdd vdd pch w=2u l=180n
CT684 t684 0 0.1f
M1751 nw192 nw189 t684 0 nch w=1u l=180n
M1752 t684 nw186 0 0 nch w=1u l=180n
Cnw192 nw192 0 2f
M1753 nw193 nw191 vdd vdd pch w=2u l=180n
M1754 nw193 nw192 vdd vdd pch w=2u l=180n
CT685 t685 0 0.1f
M1755 nw193 nw191 t685 0 nch w=1u l=180n
M1756 t685 nw192 0 0 nch w=1u l=180n
Cnw193 nw193 0 2f
CT686 t686 0 0.1f
M1757 t686 nw190 vdd vdd pch w=2u l=180n
M1758 t686 nw190 0 0 nch w=1u l=180n
M1759 ns27 t686 vdd vdd pch w=2u l=180n
M1760 ns27 t686 0 0 nch w=1u l=180n
Cns27 ns27 0 2f
CT687 t687 0 0.1f
CT688 t688 0 0.1f
CT689 t689 0 0.1f
M1761 t687 nw188 vdd vdd pch w=2u l=180n
M1762 t687 nw190 vdd vdd pch w=2u l=180n
CT690 t690 0 0.1f
M1763 t687 nw188 t690 0 nch w=1u l=180n
M1764 t690 nw190 0 0 nch w=1u l=180n
M1765 t688 nw188 vdd vdd pch w=2u l=180n
M1766 t688 t687 vdd vdd pch w=2u l=180n
CT691 t691 0 0.1f
M1767 t688 nw188 t691 0 nch w=1u l=180n
M1768 t691 t687 0 0 nch w=1u l=180n
M1769 t689 nw190 vdd vdd pch w=2u l=180n
M1770 t689 t687 vdd vdd pch w=2u l=180n
CT692 t692 0 0.1f
M1771 t689 nw190 t692 0 nch w=1u l=180n
M1772 t692 t687 0 0 nch w=1u l=180n
M1773 nw195 t688 vdd vdd pch w=2u l=180n
M1774 nw195 t689 vdd vdd pch w=2u l=180n
CT693 t693 0 0.1f
M1775 nw195 t688 t693 0 nch w=1u l=180n
M1776 t693 t689 0 0 nch w=1u l=180n
Cnw195 nw195 0 2f
CT694 t694 0 0.1f
CT695 t695 0 0.1f
CT696 t696 0 0.1f
M1777 t694 na28 vdd vdd pch w=2u l=180n
M1778 t694 nb28 vdd vdd pch w=2u l=180n
CT697 t697 0 0.1f
M1779 t694 na28 t697 0 nch w=1u l=180n
M1780 t697 nb28 0 0 nch w=1u l=180n
M1781 t695 na28 vdd vdd pch w=2u l=180n
M1782 t695 t694 vdd vdd pch w=2u l=180n
CT698 t698 0 0.1f
M1783 t695 na28 t698 0 nch w=1u l=180n
M1784 t698 t694 0 0 nch w=1u l=180n
M1785 t696 nb28 vdd vdd pch w=2u l=180n
M1786 t696 t694 vdd vdd pch w=2u l=180n
CT699 t699 0 0.1f
M1787 t696 nb28 t699 0 nch w=1u l=180n
M1788 t699 t694 0 0 nch w=1u l=180n
M1789 nw196 t695 vdd vdd pch w=2u l=180n
M1790 nw196 t696 vdd vdd pch w=2u l=180n
CT700 t700 0 0.1f
M1791 nw196 t695 t700 0 nch w=1u l=180n
M1792 t700 t696 0 0 nch w=1u l=180n
Cnw196 nw196 0 2f
CT701 t701 0 0.1f
CT702 t702 0 0.1f
CT703 t703 0 0.1f
M1793 t701 nw196 vdd vdd pch w=2u l=180n
M1794 t701 nw193 vdd vdd pch w=2u l=180n
CT704 t704 0 0.1f
M1795 t701 nw196 t704 0 nch w=1u l=180n
M1796 t704 nw193 0 0 nch w=1u l=180n
M1797 t702 nw196 vdd vdd pch w=2u l=180n
M1798 t702 t701 vdd vdd pch w=2u l=180n
CT705 t705 0 0.1f
M1799 t702 nw196 t705 0 nch w=1u l=180n
M1800 t705 t701 0 0 nch w=1u l=180n
M1801 t703 nw193 vdd vdd pch w=2u l=180n
M1802 t703 t701 vdd vdd pch w=2u l=180n
CT706 t706 0 0.1f
M1803 t703 nw193 t706 0 nch w=1u l=180n
M1804 t706 t701 0 0 nch w=1u l=180n
M1805 nw197 t702 vdd vdd pch w=2u l=180n
M1806 nw197 t703 vdd vdd pch w=2u l=180n
CT707 t707 0 0.1f
M1807 nw197 t702 t707 0 nch w=1u l=180n
M1808 t707 t703 0 0 nch w=1u l=180n
Cnw197 nw197 0 2f
M1809 nw198 na28 vdd vdd pch w=2u l=180n
M1810 nw198 nb28 vdd vdd pch w=2u l=180n
CT708 t708 0 0.1f
M1811 nw198 na28 t708 0 nch w=1u l=180n
M1812 t708 nb28 0 0 nch w=1u l=180n
Cnw198 nw198 0 2f
M1813 nw199 nw196 vdd vdd pch w=2u l=180n
M1814 nw199 nw193 vdd vdd pch w=2u l=180n
CT709 t709 0 0.1f
M1815 nw199 nw196 t709 0 nch w=1u l=180n
M1816 t709 nw193 0 0 nch w=1u l=180n
Cnw199 nw199 0 2f
M1817 nw200 nw198 vdd vdd pch w=2u l=180n
M1818 nw200 nw199 vdd vdd pch w=2u l=180n
CT710 t710 0 0.1f
M1819 nw200 nw198 t710 0 nch w=1u l=180n
M1820 t710 nw199 0 0 nch w=1u l=180n
Cnw200 nw200 0 2f
CT711 t711 0 0.1f
M1821 t711 nw197 vdd vdd pch w=2u l=180n
M1822 t711 nw197 0 0 nch w=1u l=180n
M1823 ns28 t711 vdd vdd pch w=2u l=180n
M1824 ns28 t711 0 0 nch w=1u l=180n
Cns28 ns28 0 2f
CT712 t712 0 0.1f
CT713 t713 0 0.1f
CT714 t714 0 0.1f
M1825 t712 nw195 vdd vdd pch w=2u l=180n
M1826 t712 nw197 vdd vdd pch w=2u l=180n
CT715 t715 0 0.1f
M1827 t712 nw195 t715 0 nch w=1u l=180n
M1828 t715 nw197 0 0 nch w=1u l=180n
M1829 t713 nw195 vdd vdd pch w=2u l=180n
M1830 t713 t712 vdd vdd pch w=2u l=180n
CT716 t716 0 0.1f
M1831 t713 nw195 t716 0 nch w=1u l=180n
M1832 t716 t712 0 0 nch w=1u l=180n
M1833 t714 nw197 vdd vdd pch w=2u l=180n
M1834 t714 t712 vdd vdd pch w=2u l=180n
CT717 t717 0 0.1f
M1835 t714 nw197 t717 0 nch w=1u l=180n
M1836 t717 t712 0 0 nch w=1u l=180n
M1837 nw202 t713 vdd vdd pch w=2u l=180n
M1838 nw202 t714 vdd vdd pch w=2u l=180n
CT718 t718 0 0.1f
M1839 nw202 t713 t718 0 nch w=1u l=180n
M1840 t718 t714 0 0 nch w=1u l=180n
Cnw202 nw202 0 2f
CT719 t719 0 0.1f
CT720 t720 0 0.1f
CT721 t721 0 0.1f
M1841 t719 na29 vdd vdd pch w=2u l=180n
M1842 t719 nb29 vdd vdd pch w=2u l=180n
CT722 t722 0 0.1f
M1843 t719 na29 t722 0 nch w=1u l=180n
M1844 t722 nb29 0 0 nch w=1u l=180n
M1845 t720 na29 vdd vdd pch w=2u l=180n
M1846 t720 t719 vdd vdd pch w=2u l=180n
CT723 t723 0 0.1f
M1847 t720 na29 t723 0 nch w=1u l=180n
M1848 t723 t719 0 0 nch w=1u l=180n
M1849 t721 nb29 vdd vdd pch w=2u l=180n
M1850 t721 t719 vdd vdd pch w=2u l=180n
CT724 t724 0 0.1f
M1851 t721 nb29 t724 0 nch w=1u l=180n
M1852 t724 t719 0 0 nch w=1u l=180n
M1853 nw203 t720 vdd vdd pch w=2u l=180n
M1854 nw203 t721 vdd vdd pch w=2u l=180n
CT725 t725 0 0.1f
M1855 nw203 t720 t725 0 nch w=1u l=180n
M1856 t725 t721 0 0 nch w=1u l=180n
Cnw203 nw203 0 2f
CT726 t726 0 0.1f
CT727 t727 0 0.1f
CT728 t728 0 0.1f
M1857 t726 nw203 vdd vdd pch w=2u l=180n
M1858 t726 nw200 vdd vdd pch w=2u l=180n
CT729 t729 0 0.1f
M1859 t726 nw203 t729 0 nch w=1u l=180n
M1860 t729 nw200 0 0 nch w=1u l=180n
M1861 t727 nw203 vdd vdd pch w=2u l=180n
M1862 t727 t726 vdd vdd pch w=2u l=180n
CT730 t730 0 0.1f
M1863 t727 nw203 t730 0 nch w=1u l=180n
M1864 t730 t726 0 0 nch w=1u l=180n
M1865 t728 nw200 vdd vdd pch w=2u l=180n
M1866 t728 t726 vdd vdd pch w=2u l=180n
CT731 t731 0 0.1f
M1867 t728 nw200 t731 0 nch w=1u l=180n
M1868 t731 t726 0 0 nch w=1u l=180n
M1869 nw204 t727 vdd vdd pch w=2u l=180n
M1870 nw204 t728 vdd vdd pch w=2u l=180n
CT732 t732 0 0.1f
M1871 nw204 t727 t732 0 nch w=1u l=180n
M1872 t732 t728 0 0 nch w=1u l=180n
Cnw204 nw204 0 2f
M1873 nw205 na29 vdd vdd pch w=2u l=180n
M1874 nw205 nb29 vdd vdd pch w=2u l=180n
CT733 t733 0 0.1f
M1875 nw205 na29 t733 0 nch w=1u l=180n
M1876 t733 nb29 0 0 nch w=1u l=180n
Cnw205 nw205 0 2f
M1877 nw206 nw203 vdd vdd pch w=2u l=180n
M1878 nw206 nw200 vdd vdd pch w=2u l=180n
CT734 t734 0 0.1f
M1879 nw206 nw203 t734 0 nch w=1u l=180n
M1880 t734 nw200 0 0 nch w=1u l=180n
Cnw206 nw206 0 2f
M1881 nw207 nw205 vdd vdd pch w=2u l=180n
M1882 nw207 nw206 vdd vdd pch w=2u l=180n
CT735 t735 0 0.1f
M1883 nw207 nw205 t735 0 nch w=1u l=180n
M1884 t735 nw206 0 0 nch w=1u l=180n
Cnw207 nw207 0 2f
CT736 t736 0 0.1f
M1885 t736 nw204 vdd vdd pch w=2u l=180n
M1886 t736 nw204 0 0 nch w=1u l=180n
M1887 ns29 t736 vdd vdd pch w=2u l=180n
M1888 ns29 t736 0 0 nch w=1u l=180n
Cns29 ns29 0 2f
CT737 t737 0 0.1f
CT738 t738 0 0.1f
CT739 t739 0 0.1f
M1889 t737 nw202 vdd vdd pch w=2u l=180n
M1890 t737 nw204 vdd vdd pch w=2u l=180n
CT740 t740 0 0.1f
M1891 t737 nw202 t740 0 nch w=1u l=180n
M1892 t740 nw204 0 0 nch w=1u l=180n
M1893 t738 nw202 vdd vdd pch w=2u l=180n
M1894 t738 t737 vdd vdd pch w=2u l=180n
CT741 t741 0 0.1f
M1895 t738 nw202 t741 0 nch w=1u l=180n
M1896 t741 t737 0 0 nch w=1u l=180n
M1897 t739 nw204 vdd vdd pch w=2u l=180n
M1898 t739 t737 vdd vdd pch w=2u l=180n
CT742 t742 0 0.1f
M1899 t739 nw204 t742 0 nch w=1u l=180n
M1900 t742 t737 0 0 nch w=1u l=180n
M1901 nw209 t738 vdd vdd pch w=2u l=180n
M1902 nw209 t739 vdd vdd pch w=2u l=180n
CT743 t743 0 0.1f
M1903 nw209 t738 t743 0 nch w=1u l=180n
M1904 t743 t739 0 0 nch w=1u l=180n
Cnw209 nw209 0 2f
CT744 t744 0 0.1f
CT745 t745 0 0.1f
CT746 t746 0 0.1f
M1905 t744 na30 vdd vdd pch w=2u l=180n
M1906 t744 nb30 vdd vdd pch w=2u l=180n
CT747 t747 0 0.1f
M1907 t744 na30 t747 0 nch w=1u l=180n
M1908 t747 nb30 0 0 nch w=1u l=180n
M1909 t745 na30 vdd vdd pch w=2u l=180n
M1910 t745 t744 vdd vdd pch w=2u l=180n
CT748 t748 0 0.1f
M1911 t745 na30 t748 0 nch w=1u l=180n
M1912 t748 t744 0 0 nch w=1u l=180n
M1913 t746 nb30 vdd vdd pch w=2u l=180n
M1914 t746 t744 vdd vdd pch w=2u l=180n
CT749 t749 0 0.1f
M1915 t746 nb30 t749 0 nch w=1u l=180n
M1916 t749 t744 0 0 nch w=1u l=180n
M1917 nw210 t745 vdd vdd pch w=2u l=180n
M1918 nw210 t746 vdd vdd pch w=2u l=180n
CT750 t750 0 0.1f
M1919 nw210 t745 t750 0 nch w=1u l=180n
M1920 t750 t746 0 0 nch w=1u l=180n
Cnw210 nw210 0 2f
CT751 t751 0 0.1f
CT752 t752 0 0.1f
CT753 t753 0 0.1f
M1921 t751 nw210 vdd vdd pch w=2u l=180n
M1922 t751 nw207 vdd vdd pch w=2u l=180n
CT754 t754 0 0.1f
M1923 t751 nw210 t754 0 nch w=1u l=180n
M1924 t754 nw207 0 0 nch w=1u l=180n
M1925 t752 nw210 vdd vdd pch w=2u l=180n
M1926 t752 t751 vdd vdd pch w=2u l=180n
CT755 t755 0 0.1f
M1927 t752 nw210 t755 0 nch w=1u l=180n
M1928 t755 t751 0 0 nch w=1u l=180n
M1929 t753 nw207 vdd vdd pch w=2u l=180n
M1930 t753 t751 vdd vdd pch w=2u l=180n
CT756 t756 0 0.1f
M1931 t753 nw207 t756 0 nch w=1u l=180n
M1932 t756 t751 0 0 nch w=1u l=180n
M1933 nw211 t752 vdd vdd pch w=2u l=180n
M1934 nw211 t753 vdd vdd pch w=2u l=180n
CT757 t757 0 0.1f
M1935 nw211 t752 t757 0 nch w=1u l=180n
M1936 t757 t753 0 0 nch w=1u l=180n
Cnw211 nw211 0 2f
M1937 nw212 na30 vdd vdd pch w=2u l=180n
M1938 nw212 nb30 vdd vdd pch w=2u l=180n
CT758 t758 0 0.1f
M1939 nw212 na30 t758 0 nch w=1u l=180n
M1940 t758 nb30 0 0 nch w=1u l=180n
Cnw212 nw212 0 2f
M1941 nw213 nw210 vdd vdd pch w=2u l=180n
M1942 nw213 nw207 vdd vdd pch w=2u l=180n
CT759 t759 0 0.1f
M1943 nw213 nw210 t759 0 nch w=1u l=180n
M1944 t759 nw207 0 0 nch w=1u l=180n
Cnw213 nw213 0 2f
M1945 nw214 nw212 vdd vdd pch w=2u l=180n
M1946 nw214 nw213 vdd vdd pch w=2u l=180n
CT760 t760 0 0.1f
M1947 nw214 nw212 t760 0 nch w=1u l=180n
M1948 t760 nw213 0 0 nch w=1u l=180n
Cnw214 nw214 0 2f
CT761 t761 0 0.1f
M1949 t761 nw211 vdd vdd pch w=2u l=180n
M1950 t761 nw211 0 0 nch w=1u l=180n
M1951 ns30 t761 vdd vdd pch w=2u l=180n
M1952 ns30 t761 0 0 nch w=1u l=180n
Cns30 ns30 0 2f
CT762 t762 0 0.1f
CT763 t763 0 0.1f
CT764 t764 0 0.1f
M1953 t762 nw209 vdd vdd pch w=2u l=180n
M1954 t762 nw211 vdd vdd pch w=2u l=180n
CT765 t765 0 0.1f
M1955 t762 nw209 t765 0 nch w=1u l=180n
M1956 t765 nw211 0 0 nch w=1u l=180n
M1957 t763 nw209 vdd vdd pch w=2u l=180n
M1958 t763 t762 vdd vdd pch w=2u l=180n
CT766 t766 0 0.1f
M1959 t763 nw209 t766 0 nch w=1u l=180n
M1960 t766 t762 0 0 nch w=1u l=180n
M1961 t764 nw211 vdd vdd pch w=2u l=180n
M1962 t764 t762 vdd vdd pch w=2u l=180n
CT767 t767 0 0.1f
M1963 t764 nw211 t767 0 nch w=1u l=180n
M1964 t767 t762 0 0 nch w=1u l=180n
M1965 nw216 t763 vdd vdd pch w=2u l=180n
M1966 nw216 t764 vdd vdd pch w=2u l=180n
CT768 t768 0 0.1f
M1967 nw216 t763 t768 0 nch w=1u l=180n
M1968 t768 t764 0 0 nch w=1u l=180n
Cnw216 nw216 0 2f
CT769 t769 0 0.1f
CT770 t770 0 0.1f
CT771 t771 0 0.1f
M1969 t769 na31 vdd vdd pch w=2u l=180n
M1970 t769 nb31 vdd vdd pch w=2u l=180n
CT772 t772 0 0.1f
M1971 t769 na31 t772 0 nch w=1u l=180n
M1972 t772 nb31 0 0 nch w=1u l=180n
M1973 t770 na31 vdd vdd pch w=2u l=180n
M1974 t770 t769 vdd vdd pch w=2u l=180n
CT773 t773 0 0.1f
M1975 t770 na31 t773 0 nch w=1u l=180n
M1976 t773 t769 0 0 nch w=1u l=180n
M1977 t771 nb31 vdd vdd pch w=2u l=180n
M1978 t771 t769 vdd vdd pch w=2u l=180n
CT774 t774 0 0.1f
M1979 t771 nb31 t774 0 nch w=1u l=180n
M1980 t774 t769 0 0 nch w=1u l=180n
M1981 nw217 t770 vdd vdd pch w=2u l=180n
M1982 nw217 t771 vdd vdd pch w=2u l=180n
CT775 t775 0 0.1f
M1983 nw217 t770 t775 0 nch w=1u l=180n
M1984 t775 t771 0 0 nch w=1u l=180n
Cnw217 nw217 0 2f
CT776 t776 0 0.1f
CT777 t777 0 0.1f
CT778 t778 0 0.1f
M1985 t776 nw217 vdd vdd pch w=2u l=180n
M1986 t776 nw214 vdd vdd pch w=2u l=180n
CT779 t779 0 0.1f
M1987 t776 nw217 t779 0 nch w=1u l=180n
M1988 t779 nw214 0 0 nch w=1u l=180n
M1989 t777 nw217 vdd vdd pch w=2u l=180n
M1990 t777 t776 vdd vdd pch w=2u l=180n
CT780 t780 0 0.1f
M1991 t777 nw217 t780 0 nch w=1u l=180n
M1992 t780 t776 0 0 nch w=1u l=180n
M1993 t778 nw214 vdd vdd pch w=2u l=180n
M1994 t778 t776 vdd vdd pch w=2u l=180n
CT781 t781 0 0.1f
M1995 t778 nw214 t781 0 nch w=1u l=180n
M1996 t781 t776 0 0 nch w=1u l=180n
M1997 nw218 t777 vdd vdd pch w=2u l=180n
M1998 nw218 t778 vdd vdd pch w=2u l=180n
CT782 t782 0 0.1f
M1999 nw218 t777 t782 0 nch w=1u l=180n
M2000 t782 t778 0 0 nch w=1u l=180n
Cnw218 nw218 0 2f
M2001 nw219 na31 vdd vdd pch w=2u l=180n
M2002 nw219 nb31 vdd vdd pch w=2u l=180n
CT783 t783 0 0.1f
M2003 nw219 na31 t783 0 nch w=1u l=180n
M2004 t783 nb31 0 0 nch w=1u l=180n
Cnw219 nw219 0 2f
M2005 nw220 nw217 vdd vdd pch w=2u l=180n
M2006 nw220 nw214 vdd vdd pch w=2u l=180n
CT784 t784 0 0.1f
M2007 nw220 nw217 t784 0 nch w=1u l=180n
M2008 t784 nw214 0 0 nch w=1u l=180n
Cnw220 nw220 0 2f
M2009 nw221 nw219 vdd vdd pch w=2u l=180n
M2010 nw221 nw220 vdd vdd pch w=2u l=180n
CT785 t785 0 0.1f
M2011 nw221 nw219 t785 0 nch w=1u l=180n
M2012 t785 nw220 0 0 nch w=1u l=180n
Cnw221 nw221 0 2f
CT786 t786 0 0.1f
M2013 t786 nw218 vdd vdd pch w=2u l=180n
M2014 t786 nw218 0 0 nch w=1u l=180n
M2015 ns31 t786 vdd vdd pch w=2u l=180n
M2016 ns31 t786 0 0 nch w=1u l=180n
Cns31 ns31 0 2f
CT787 t787 0 0.1f
CT788 t788 0 0.1f
CT789 t789 0 0.1f
M2017 t787 nw216 vdd vdd pch w=2u l=180n
M2018 t787 nw218 vdd vdd pch w=2u l=180n
CT790 t790 0 0.1f
M2019 t787 nw216 t790 0 nch w=1u l=180n
M2020 t790 nw218 0 0 nch w=1u l=180n
M2021 t788 nw216 vdd vdd pch w=2u l=180n
M2022 t788 t787 vdd vdd pch w=2u l=180n
CT791 t791 0 0.1f
M2023 t788 nw216 t791 0 nch w=1u l=180n
M2024 t791 t787 0 0 nch w=1u l=180n
M2025 t789 nw218 vdd vdd pch w=2u l=180n
M2026 t789 t787 vdd vdd pch w=2u l=180n
CT792 t792 0 0.1f
M2027 t789 nw218 t792 0 nch w=1u l=180n
M2028 t792 t787 0 0 nch w=1u l=180n
M2029 nw223 t788 vdd vdd pch w=2u l=180n
M2030 nw223 t789 vdd vdd pch w=2u l=180n
CT793 t793 0 0.1f
M2031 nw223 t788 t793 0 nch w=1u l=180n
M2032 t793 t789 0 0 nch w=1u l=180n
Cnw223 nw223 0 2f
CT794 t794 0 0.1f
CT795 t795 0 0.1f
CT796 t796 0 0.1f
M2033 t794 na31 vdd vdd pch w=2u l=180n
M2034 t794 nb31 vdd vdd pch w=2u l=180n
CT797 t797 0 0.1f
M2035 t794 na31 t797 0 nch w=1u l=180n
M2036 t797 nb31 0 0 nch w=1u l=180n
M2037 t795 na31 vdd vdd pch w=2u l=180n
M2038 t795 t794 vdd vdd pch w=2u l=180n
CT798 t798 0 0.1f
M2039 t795 na31 t798 0 nch w=1u l=180n
M2040 t798 t794 0 0 nch w=1u l=180n
M2041 t796 nb31 vdd vdd pch w=2u l=180n
M2042 t796 t794 vdd vdd pch w=2u l=180n
CT799 t799 0 0.1f
M2043 t796 nb31 t799 0 nch w=1u l=180n
M2044 t799 t794 0 0 nch w=1u l=180n
CT800 t800 0 0.1f
M2045 t800 t795 vdd vdd pch w=2u l=180n
M2046 t800 t796 vdd vdd pch w=2u l=180n
CT801 t801 0 0.1f
M2047 t800 t795 t801 0 nch w=1u l=180n
M2048 t801 t796 0 0 nch w=1u l=180n
M2049 nw224 t800 vdd vdd pch w=2u l=180n
M2050 nw224 t800 0 0 nch w=1u l=180n
Cnw224 nw224 0 2f
M2051 nw225 nb31 vdd vdd pch w=2u l=180n
M2052 nw225 nb31 0 0 nch w=1u l=180n
Cnw225 nw225 0 2f
CT802 t802 0 0.1f
M2053 t802 na31 vdd vdd pch w=2u l=180n
M2054 t802 nw225 vdd vdd pch w=2u l=180n
CT803 t803 0 0.1f
M2055 t802 na31 t803 0 nch w=1u l=180n
M2056 t803 nw225 0 0 nch w=1u l=180n
M2057 nw226 t802 vdd vdd pch w=2u l=180n
M2058 nw226 t802 0 0 nch w=1u l=180n
Cnw226 nw226 0 2f
CT804 t804 0 0.1f
CT805 t805 0 0.1f
CT806 t806 0 0.1f
M2059 t804 na30 vdd vdd pch w=2u l=180n
M2060 t804 nb30 vdd vdd pch w=2u l=180n
CT807 t807 0 0.1f
M2061 t804 na30 t807 0 nch w=1u l=180n
M2062 t807 nb30 0 0 nch w=1u l=180n
M2063 t805 na30 vdd vdd pch w=2u l=180n
M2064 t805 t804 vdd vdd pch w=2u l=180n
CT808 t808 0 0.1f
M2065 t805 na30 t808 0 nch w=1u l=180n
M2066 t808 t804 0 0 nch w=1u l=180n
M2067 t806 nb30 vdd vdd pch w=2u l=180n
M2068 t806 t804 vdd vdd pch w=2u l=180n
CT809 t809 0 0.1f
M2069 t806 nb30 t809 0 nch w=1u l=180n
M2070 t809 t804 0 0 nch w=1u l=180n
CT810 t810 0 0.1f
M2071 t810 t805 vdd vdd pch w=2u l=180n
M2072 t810 t806 vdd vdd pch w=2u l=180n
CT811 t811 0 0.1f
M2073 t810 t805 t811 0 nch w=1u l=180n
M2074 t811 t806 0 0 nch w=1u l=180n
M2075 nw227 t810 vdd vdd pch w=2u l=180n
M2076 nw227 t810 0 0 nch w=1u l=180n
Cnw227 nw227 0 2f
M2077 nw228 nb30 vdd vdd pch w=2u l=180n
M2078 nw228 nb30 0 0 nch w=1u l=180n
Cnw228 nw228 0 2f
CT812 t812 0 0.1f
M2079 t812 na30 vdd vdd pch w=2u l=180n
M2080 t812 nw228 vdd vdd pch w=2u l=180n
CT813 t813 0 0.1f
M2081 t812 na30 t813 0 nch w=1u l=180n
M2082 t813 nw228 0 0 nch w=1u l=180n
M2083 nw229 t812 vdd vdd pch w=2u l=180n
M2084 nw229 t812 0 0 nch w=1u l=180n
Cnw229 nw229 0 2f
CT814 t814 0 0.1f
M2085 t814 nw224 vdd vdd pch w=2u l=180n
M2086 t814 nw229 vdd vdd pch w=2u l=180n
CT815 t815 0 0.1f
M2087 t814 nw224 t815 0 nch w=1u l=180n
M2088 t815 nw229 0 0 nch w=1u l=180n
M2089 nw230 t814 vdd vdd pch w=2u l=180n
M2090 nw230 t814 0 0 nch w=1u l=180n
Cnw230 nw230 0 2f
CT816 t816 0 0.1f
M2091 t816 nw226 0 0 nch w=1u l=180n
M2092 t816 nw230 0 0 nch w=1u l=180n
CT817 t817 0 0.1f
M2093 t817 nw226 vdd vdd pch w=2u l=180n
M2094 t816 nw230 t817 vdd pch w=2u l=180n
M2095 nw231 t816 vdd vdd pch w=2u l=180n
M2096 nw231 t816 0 0 nch w=1u l=180n
Cnw231 nw231 0 2f
CT818 t818 0 0.1f
M2097 t818 nw224 vdd vdd pch w=2u l=180n
M2098 t818 nw227 vdd vdd pch w=2u l=180n
CT819 t819 0 0.1f
M2099 t818 nw224 t819 0 nch w=1u l=180n
M2100 t819 nw227 0 0 nch w=1u l=180n
M2101 nw232 t818 vdd vdd pch w=2u l=180n
M2102 nw232 t818 0 0 nch w=1u l=180n
Cnw232 nw232 0 2f
CT820 t820 0 0.1f
CT821 t821 0 0.1f
CT822 t822 0 0.1f
M2103 t820 na29 vdd vdd pch w=2u l=180n
M2104 t820 nb29 vdd vdd pch w=2u l=180n
CT823 t823 0 0.1f
M2105 t820 na29 t823 0 nch w=1u l=180n
M2106 t823 nb29 0 0 nch w=1u l=180n
M2107 t821 na29 vdd vdd pch w=2u l=180n
M2108 t821 t820 vdd vdd pch w=2u l=180n
CT824 t824 0 0.1f
M2109 t821 na29 t824 0 nch w=1u l=180n
M2110 t824 t820 0 0 nch w=1u l=180n
M2111 t822 nb29 vdd vdd pch w=2u l=180n
M2112 t822 t820 vdd vdd pch w=2u l=180n
CT825 t825 0 0.1f
M2113 t822 nb29 t825 0 nch w=1u l=180n
M2114 t825 t820 0 0 nch w=1u l=180n
CT826 t826 0 0.1f
M2115 t826 t821 vdd vdd pch w=2u l=180n
M2116 t826 t822 vdd vdd pch w=2u l=180n
CT827 t827 0 0.1f
M2117 t826 t821 t827 0 nch w=1u l=180n
M2118 t827 t822 0 0 nch w=1u l=180n
M2119 nw233 t826 vdd vdd pch w=2u l=180n
M2120 nw233 t826 0 0 nch w=1u l=180n
Cnw233 nw233 0 2f
M2121 nw234 nb29 vdd vdd pch w=2u l=180n
M2122 nw234 nb29 0 0 nch w=1u l=180n
Cnw234 nw234 0 2f
CT828 t828 0 0.1f
M2123 t828 na29 vdd vdd pch w=2u l=180n
M2124 t828 nw234 vdd vdd pch w=2u l=180n
CT829 t829 0 0.1f
M2125 t828 na29 t829 0 nch w=1u l=180n
M2126 t829 nw234 0 0 nch w=1u l=180n
M2127 nw235 t828 vdd vdd pch w=2u l=180n
M2128 nw235 t828 0 0 nch w=1u l=180n
Cnw235 nw235 0 2f
CT830 t830 0 0.1f
M2129 t830 nw232 vdd vdd pch w=2u l=180n
M2130 t830 nw235 vdd vdd pch w=2u l=180n
CT831 t831 0 0.1f
M2131 t830 nw232 t831 0 nch w=1u l=180n
M2132 t831 nw235 0 0 nch w=1u l=180n
M2133 nw236 t830 vdd vdd pch w=2u l=180n
M2134 nw236 t830 0 0 nch w=1u l=180n
Cnw236 nw236 0 2f
CT832 t832 0 0.1f
M2135 t832 nw231 0 0 nch w=1u l=180n
M2136 t832 nw236 0 0 nch w=1u l=180n
CT833 t833 0 0.1f
M2137 t833 nw231 vdd vdd pch w=2u l=180n
M2138 t832 nw236 t833 vdd pch w=2u l=180n
M2139 nw237 t832 vdd vdd pch w=2u l=180n
M2140 nw237 t832 0 0 nch w=1u l=180n
Cnw237 nw237 0 2f
CT834 t834 0 0.1f
M2141 t834 nw232 vdd vdd pch w=2u l=180n
M2142 t834 nw233 vdd vdd pch w=2u l=180n
CT835 t835 0 0.1f
M2143 t834 nw232 t835 0 nch w=1u l=180n
M2144 t835 nw233 0 0 nch w=1u l=180n
M2145 nw238 t834 vdd vdd pch w=2u l=180n
M2146 nw238 t834 0 0 nch w=1u l=180n
Cnw238 nw238 0 2f
CT836 t836 0 0.1f
CT837 t837 0 0.1f
CT838 t838 0 0.1f
M2147 t836 na28 vdd vdd pch w=2u l=180n
M2148 t836 nb28 vdd vdd pch w=2u l=180n
CT839 t839 0 0.1f
M2149 t836 na28 t839 0 nch w=1u l=180n
M2150 t839 nb28 0 0 nch w=1u l=180n
M2151 t837 na28 vdd vdd pch w=2u l=180n
M2152 t837 t836 vdd vdd pch w=2u l=180n
CT840 t840 0 0.1f
M2153 t837 na28 t840 0 nch w=1u l=180n
M2154 t840 t836 0 0 nch w=1u l=180n
M2155 t838 nb28 vdd vdd pch w=2u l=180n
M2156 t838 t836 vdd vdd pch w=2u l=180n
CT841 t841 0 0.1f
M2157 t838 nb28 t841 0 nch w=1u l=180n
M2158 t841 t836 0 0 nch w=1u l=180n
CT842 t842 0 0.1f
M2159 t842 t837 vdd vdd pch w=2u l=180n
M2160 t842 t838 vdd vdd pch w=2u l=180n
CT843 t843 0 0.1f
M2161 t842 t837 t843 0 nch w=1u l=180n
M2162 t843 t838 0 0 nch w=1u l=180n
M2163 nw239 t842 vdd vdd pch w=2u l=180n
M2164 nw239 t842 0 0 nch w=1u l=180n
Cnw239 nw239 0 2f
M2165 nw240 nb28 vdd vdd pch w=2u l=180n
M2166 nw240 nb28 0 0 nch w=1u l=180n
Cnw240 nw240 0 2f
CT844 t844 0 0.1f
M2167 t844 na28 vdd vdd pch w=2u l=180n
M2168 t844 nw240 vdd vdd pch w=2u l=180n
CT845 t845 0 0.1f
M2169 t844 na28 t845 0 nch w=1u l=180n
M2170 t845 nw240 0 0 nch w=1u l=180n
M2171 nw241 t844 vdd vdd pch w=2u l=180n
M2172 nw241 t844 0 0 nch w=1u l=180n
Cnw241 nw241 0 2f
CT846 t846 0 0.1f
M2173 t846 nw238 vdd vdd pch w=2u l=180n
M2174 t846 nw241 vdd vdd pch w=2u l=180n
CT847 t847 0 0.1f
M2175 t846 nw238 t847 0 nch w=1u l=180n
M2176 t847 nw241 0 0 nch w=1u l=180n
M2177 nw242 t846 vdd vdd pch w=2u l=180n
M2178 nw242 t846 0 0 nch w=1u l=180n
Cnw242 nw242 0 2f
CT848 t848 0 0.1f
M2179 t848 nw237 0 0 nch w=1u l=180n
M2180 t848 nw242 0 0 nch w=1u l=180n
CT849 t849 0 0.1f
M2181 t849 nw237 vdd vdd pch w=2u l=180n
M2182 t848 nw242 t849 vdd pch w=2u l=180n
M2183 nw243 t848 vdd vdd pch w=2u l=180n
M2184 nw243 t848 0 0 nch w=1u l=180n
Cnw243 nw243 0 2f
CT850 t850 0 0.1f
M2185 t850 nw238 vdd vdd pch w=2u l=180n
M2186 t850 nw239 vdd vdd pch w=2u l=180n
CT851 t851 0 0.1f
M2187 t850 nw238 t851 0 nch w=1u l=180n
M2188 t851 nw239 0 0 nch w=1u l=180n
M2189 nw244 t850 vdd vdd pch w=2u l=180n
M2190 nw244 t850 0 0 nch w=1u l=180n
Cnw244 nw244 0 2f
CT852 t852 0 0.1f
CT853 t853 0 0.1f
CT854 t854 0 0.1f
M2191 t852 na27 vdd vdd pch w=2u l=180n
M2192 t852 nb27 vdd vdd pch w=2u l=180n
CT855 t855 0 0.1f
M2193 t852 na27 t855 0 nch w=1u l=180n
M2194 t855 nb27 0 0 nch w=1u l=180n
M2195 t853 na27 vdd vdd pch w=2u l=180n
M2196 t853 t852 vdd vdd pch w=2u l=180n
CT856 t856 0 0.1f
M2197 t853 na27 t856 0 nch w=1u l=180n
M2198 t856 t852 0 0 nch w=1u l=180n
M2199 t854 nb27 vdd vdd pch w=2u l=180n
M2200 t854 t852 vdd vdd pch w=2u l=180n
CT857 t857 0 0.1f
M2201 t854 nb27 t857 0 nch w=1u l=180n
M2202 t857 t852 0 0 nch w=1u l=180n
CT858 t858 0 0.1f
M2203 t858 t853 vdd vdd pch w=2u l=180n
M2204 t858 t854 vdd vdd pch w=2u l=180n
CT859 t859 0 0.1f
M2205 t858 t853 t859 0 nch w=1u l=180n
M2206 t859 t854 0 0 nch w=1u l=180n
M2207 nw245 t858 vdd vdd pch w=2u l=180n
M2208 nw245 t858 0 0 nch w=1u l=180n
Cnw245 nw245 0 2f
M2209 nw246 nb27 vdd vdd pch w=2u l=180n
M2210 nw246 nb27 0 0 nch w=1u l=180n
Cnw246 nw246 0 2f
CT860 t860 0 0.1f
M2211 t860 na27 vdd vdd pch w=2u l=180n
M2212 t860 nw246 vdd vdd pch w=2u l=180n
CT861 t861 0 0.1f
M2213 t860 na27 t861 0 nch w=1u l=180n
M2214 t861 nw246 0 0 nch w=1u l=180n
M2215 nw247 t860 vdd vdd pch w=2u l=180n
M2216 nw247 t860 0 0 nch w=1u l=180n
Cnw247 nw247 0 2f
CT862 t862 0 0.1f
M2217 t862 nw244 vdd vdd pch w=2u l=180n
M2218 t862 nw247 vdd vdd pch w=2u l=180n
CT863 t863 0 0.1f
M2219 t862 nw244 t863 0 nch w=1u l=180n
M2220 t863 nw247 0 0 nch w=1u l=180n
M2221 nw248 t862 vdd vdd pch w=2u l=180n
M2222 nw248 t862 0 0 nch w=1u l=180n
Cnw248 nw248 0 2f
CT864 t864 0 0.1f
M2223 t864 nw243 0 0 nch w=1u l=180n
M2224 t864 nw248 0 0 nch w=1u l=180n
CT865 t865 0 0.1f
M2225 t865 nw243 vdd vdd pch w=2u l=180n
M2226 t864 nw248 t865 vdd pch w=2u l=180n
M2227 nw249 t864 vdd vdd pch w=2u l=180n
M2228 nw249 t864 0 0 nch w=1u l=180n
Cnw249 nw249 0 2f
CT866 t866 0 0.1f
M2229 t866 nw244 vdd vdd pch w=2u l=180n
M2230 t866 nw245 vdd vdd pch w=2u l=180n
CT867 t867 0 0.1f
M2231 t866 nw244 t867 0 nch w=1u l=180n
M2232 t867 nw245 0 0 nch w=1u l=180n
M2233 nw250 t866 vdd vdd pch w=2u l=180n
M2234 nw250 t866 0 0 nch w=1u l=180n
Cnw250 nw250 0 2f
CT868 t868 0 0.1f
CT869 t869 0 0.1f
CT870 t870 0 0.1f
M2235 t868 na26 vdd vdd pch w=2u l=180n
M2236 t868 nb26 vdd vdd pch w=2u l=180n
CT871 t871 0 0.1f
M2237 t868 na26 t871 0 nch w=1u l=180n
M2238 t871 nb26 0 0 nch w=1u l=180n
M2239 t869 na26 vdd vdd pch w=2u l=180n
M2240 t869 t868 vdd vdd pch w=2u l=180n
CT872 t872 0 0.1f
M2241 t869 na26 t872 0 nch w=1u l=180n
M2242 t872 t868 0 0 nch w=1u l=180n
M2243 t870 nb26 vdd vdd pch w=2u l=180n
M2244 t870 t868 vdd vdd pch w=2u l=180n
CT873 t873 0 0.1f
M2245 t870 nb26 t873 0 nch w=1u l=180n
M2246 t873 t868 0 0 nch w=1u l=180n
CT874 t874 0 0.1f
M2247 t874 t869 vdd vdd pch w=2u l=180n
M2248 t874 t870 vdd vdd pch w=2u l=180n
CT875 t875 0 0.1f
M2249 t874 t869 t875 0 nch w=1u l=180n
M2250 t875 t870 0 0 nch w=1u l=180n
M2251 nw251 t874 vdd vdd pch w=2u l=180n
M2252 nw251 t874 0 0 nch w=1u l=180n
Cnw251 nw251 0 2f
M2253 nw252 nb26 vdd vdd pch w=2u l=180n
M2254 nw252 nb26 0 0 nch w=1u l=180n
Cnw252 nw252 0 2f
CT876 t876 0 0.1f
M2255 t876 na26 vdd vdd pch w=2u l=180n
M2256 t876 nw252 vdd vdd pch w=2u l=180n
CT877 t877 0 0.1f
M2257 t876 na26 t877 0 nch w=1u l=180n
M2258 t877 nw252 0 0 nch w=1u l=180n
M2259 nw253 t876 vdd vdd pch w=2u l=180n
M2260 nw253 t876 0 0 nch w=1u l=180n
Cnw253 nw253 0 2f
CT878 t878 0 0.1f
M2261 t878 nw250 vdd vdd pch w=2u l=180n
M2262 t878 nw253 vdd vdd pch w=2u l=180n
CT879 t879 0 0.1f
M2263 t878 nw250 t879 0 nch w=1u l=180n
M2264 t879 nw253 0 0 nch w=1u l=180n
M2265 nw254 t878 vdd vdd pch w=2u l=180n
M2266 nw254 t878 0 0 nch w=1u l=180n
Cnw254 nw254 0 2f
CT880 t880 0 0.1f
M2267 t880 nw249 0 0 nch w=1u l=180n
M2268 t880 nw254 0 0 nch w=1u l=180n
CT881 t881 0 0.1f
M2269 t881 nw249 vdd vdd pch w=2u l=180n
M2270 t880 nw254 t881 vdd pch w=2u l=180n
M2271 nw255 t880 vdd vdd pch w=2u l=180n
M2272 nw255 t880 0 0 nch w=1u l=180n
Cnw255 nw255 0 2f
CT882 t882 0 0.1f
M2273 t882 nw250 vdd vdd pch w=2u l=180n
M2274 t882 nw251 vdd vdd pch w=2u l=180n
CT883 t883 0 0.1f
M2275 t882 nw250 t883 0 nch w=1u l=180n
M2276 t883 nw251 0 0 nch w=1u l=180n
M2277 nw256 t882 vdd vdd pch w=2u l=180n
M2278 nw256 t882 0 0 nch w=1u l=180n
Cnw256 nw256 0 2f
CT884 t884 0 0.1f
CT885 t885 0 0.1f
CT886 t886 0 0.1f
M2279 t884 na25 vdd vdd pch w=2u l=180n
M2280 t884 nb25 vdd vdd pch w=2u l=180n
CT887 t887 0 0.1f
M2281 t884 na25 t887 0 nch w=1u l=180n
M2282 t887 nb25 0 0 nch w=1u l=180n
M2283 t885 na25 vdd vdd pch w=2u l=180n
M2284 t885 t884 vdd vdd pch w=2u l=180n
CT888 t888 0 0.1f
M2285 t885 na25 t888 0 nch w=1u l=180n
M2286 t888 t884 0 0 nch w=1u l=180n
M2287 t886 nb25 vdd vdd pch w=2u l=180n
M2288 t886 t884 vdd vdd pch w=2u l=180n
CT889 t889 0 0.1f
M2289 t886 nb25 t889 0 nch w=1u l=180n
M2290 t889 t884 0 0 nch w=1u l=180n
CT890 t890 0 0.1f
M2291 t890 t885 vdd vdd pch w=2u l=180n
M2292 t890 t886 vdd vdd pch w=2u l=180n
CT891 t891 0 0.1f
M2293 t890 t885 t891 0 nch w=1u l=180n
M2294 t891 t886 0 0 nch w=1u l=180n
M2295 nw257 t890 vdd vdd pch w=2u l=180n
M2296 nw257 t890 0 0 nch w=1u l=180n
Cnw257 nw257 0 2f
M2297 nw258 nb25 vdd vdd pch w=2u l=180n
M2298 nw258 nb25 0 0 nch w=1u l=180n
Cnw258 nw258 0 2f
CT892 t892 0 0.1f
M2299 t892 na25 vdd vdd pch w=2u l=180n
M2300 t892 nw258 vdd vdd pch w=2u l=180n
CT893 t893 0 0.1f
M2301 t892 na25 t893 0 nch w=1u l=180n
M2302 t893 nw258 0 0 nch w=1u l=180n
M2303 nw259 t892 vdd vdd pch w=2u l=180n
M2304 nw259 t892 0 0 nch w=1u l=180n
Cnw259 nw259 0 2f
CT894 t894 0 0.1f
M2305 t894 nw256 vdd vdd pch w=2u l=180n
M2306 t894 nw259 vdd vdd pch w=2u l=180n
CT895 t895 0 0.1f
M2307 t894 nw256 t895 0 nch w=1u l=180n
M2308 t895 nw259 0 0 nch w=1u l=180n
M2309 nw260 t894 vdd vdd pch w=2u l=180n
M2310 nw260 t894 0 0 nch w=1u l=180n
Cnw260 nw260 0 2f
CT896 t896 0 0.1f
M2311 t896 nw255 0 0 nch w=1u l=180n
M2312 t896 nw260 0 0 nch w=1u l=180n
CT897 t897 0 0.1f
M2313 t897 nw255 vdd vdd pch w=2u l=180n
M2314 t896 nw260 t897 vdd pch w=2u l=180n
M2315 nw261 t896 vdd vdd pch w=2u l=180n
M2316 nw261 t896 0 0 nch w=1u l=180n
Cnw261 nw261 0 2f
CT898 t898 0 0.1f
M2317 t898 nw256 vdd vdd pch w=2u l=180n
M2318 t898 nw257 vdd vdd pch w=2u l=180n
CT899 t899 0 0.1f
M2319 t898 nw256 t899 0 nch w=1u l=180n
M2320 t899 nw257 0 0 nch w=1u l=180n
M2321 nw262 t898 vdd vdd pch w=2u l=180n
M2322 nw262 t898 0 0 nch w=1u l=180n
Cnw262 nw262 0 2f
CT900 t900 0 0.1f
CT901 t901 0 0.1f
CT902 t902 0 0.1f
M2323 t900 na24 vdd vdd pch w=2u l=180n
M2324 t900 nb24 vdd vdd pch w=2u l=180n
CT903 t903 0 0.1f
M2325 t900 na24 t903 0 nch w=1u l=180n
M2326 t903 nb24 0 0 nch w=1u l=180n
M2327 t901 na24 vdd vdd pch w=2u l=180n
M2328 t901 t900 vdd vdd pch w=2u l=180n
CT904 t904 0 0.1f
M2329 t901 na24 t904 0 nch w=1u l=180n
M2330 t904 t900 0 0 nch w=1u l=180n
M2331 t902 nb24 vdd vdd pch w=2u l=180n
M2332 t902 t900 vdd vdd pch w=2u l=180n
CT905 t905 0 0.1f
M2333 t902 nb24 t905 0 nch w=1u l=180n
M2334 t905 t900 0 0 nch w=1u l=180n
CT906 t906 0 0.1f
M2335 t906 t901 vdd vdd pch w=2u l=180n
M2336 t906 t902 vdd vdd pch w=2u l=180n
CT907 t907 0 0.1f
M2337 t906 t901 t907 0 nch w=1u l=180n
M2338 t907 t902 0 0 nch w=1u l=180n
M2339 nw263 t906 vdd vdd pch w=2u l=180n
M2340 nw263 t906 0 0 nch w=1u l=180n
Cnw263 nw263 0 2f
M2341 nw264 nb24 vdd vdd pch w=2u l=180n
M2342 nw264 nb24 0 0 nch w=1u l=180n
Cnw264 nw264 0 2f
CT908 t908 0 0.1f
M2343 t908 na24 vdd vdd pch w=2u l=180n
M2344 t908 nw264 vdd vdd pch w=2u l=180n
CT909 t909 0 0.1f
M2345 t908 na24 t909 0 nch w=1u l=180n
M2346 t909 nw264 0 0 nch w=1u l=180n
M2347 nw265 t908 vdd vdd pch w=2u l=180n
M2348 nw265 t908 0 0 nch w=1u l=180n
Cnw265 nw265 0 2f
CT910 t910 0 0.1f
M2349 t910 nw262 vdd vdd pch w=2u l=180n
M2350 t910 nw265 vdd vdd pch w=2u l=180n
CT911 t911 0 0.1f
M2351 t910 nw262 t911 0 nch w=1u l=180n
M2352 t911 nw265 0 0 nch w=1u l=180n
M2353 nw266 t910 vdd vdd pch w=2u l=180n
M2354 nw266 t910 0 0 nch w=1u l=180n
Cnw266 nw266 0 2f
CT912 t912 0 0.1f
M2355 t912 nw261 0 0 nch w=1u l=180n
M2356 t912 nw266 0 0 nch w=1u l=180n
CT913 t913 0 0.1f
M2357 t913 nw261 vdd vdd pch w=2u l=180n
M2358 t912 nw266 t913 vdd pch w=2u l=180n
M2359 nw267 t912 vdd vdd pch w=2u l=180n
M2360 nw267 t912 0 0 nch w=1u l=180n
Cnw267 nw267 0 2f
CT914 t914 0 0.1f
M2361 t914 nw262 vdd vdd pch w=2u l=180n
M2362 t914 nw263 vdd vdd pch w=2u l=180n
CT915 t915 0 0.1f
M2363 t914 nw262 t915 0 nch w=1u l=180n
M2364 t915 nw263 0 0 nch w=1u l=180n
M2365 nw268 t914 vdd vdd pch w=2u l=180n
M2366 nw268 t914 0 0 nch w=1u l=180n
Cnw268 nw268 0 2f
CT916 t916 0 0.1f
CT917 t917 0 0.1f
CT918 t918 0 0.1f
M2367 t916 na23 vdd vdd pch w=2u l=180n
M2368 t916 nb23 vdd vdd pch w=2u l=180n
CT919 t919 0 0.1f
M2369 t916 na23 t919 0 nch w=1u l=180n
M2370 t919 nb23 0 0 nch w=1u l=180n
M2371 t917 na23 vdd vdd pch w=2u l=180n
M2372 t917 t916 vdd vdd pch w=2u l=180n
CT920 t920 0 0.1f
M2373 t917 na23 t920 0 nch w=1u l=180n
M2374 t920 t916 0 0 nch w=1u l=180n
M2375 t918 nb23 vdd vdd pch w=2u l=180n
M2376 t918 t916 vdd vdd pch w=2u l=180n
CT921 t921 0 0.1f
M2377 t918 nb23 t921 0 nch w=1u l=180n
M2378 t921 t916 0 0 nch w=1u l=180n
CT922 t922 0 0.1f
M2379 t922 t917 vdd vdd pch w=2u l=180n
M2380 t922 t918 vdd vdd pch w=2u l=180n
CT923 t923 0 0.1f
M2381 t922 t917 t923 0 nch w=1u l=180n
M2382 t923 t918 0 0 nch w=1u l=180n
M2383 nw269 t922 vdd vdd pch w=2u l=180n
M2384 nw269 t922 0 0 nch w=1u l=180n
Cnw269 nw269 0 2f
M2385 nw270 nb23 vdd vdd pch w=2u l=180n
M2386 nw270 nb23 0 0 nch w=1u l=180n
Cnw270 nw270 0 2f
CT924 t924 0 0.1f
M2387 t924 na23 vdd vdd pch w=2u l=180n
M2388 t924 nw270 vdd vdd pch w=2u l=180n
CT925 t925 0 0.1f
M2389 t924 na23 t925 0 nch w=1u l=180n
M2390 t925 nw270 0 0 nch w=1u l=180n
M2391 nw271 t924 vdd vdd pch w=2u l=180n
M2392 nw271 t924 0 0 nch w=1u l=180n
Cnw271 nw271 0 2f
CT926 t926 0 0.1f
M2393 t926 nw268 vdd vdd pch w=2u l=180n
M2394 t926 nw271 vdd vdd pch w=2u l=180n
CT927 t927 0 0.1f
M2395 t926 nw268 t927 0 nch w=1u l=180n
M2396 t927 nw271 0 0 nch w=1u l=180n
M2397 nw272 t926 vdd vdd pch w=2u l=180n
M2398 nw272 t926 0 0 nch w=1u l=180n
Cnw272 nw272 0 2f
CT928 t928 0 0.1f
M2399 t928 nw267 0 0 nch w=1u l=180n
M2400 t928 nw272 0 0 nch w=1u l=180n
CT929 t929 0 0.1f
M2401 t929 nw267 vdd vdd pch w=2u l=180n
M2402 t928 nw272 t929 vdd pch w=2u l=180n
M2403 nw273 t928 vdd vdd pch w=2u l=180n
M2404 nw273 t928 0 0 nch w=1u l=180n
Cnw273 nw273 0 2f
CT930 t930 0 0.1f
M2405 t930 nw268 vdd vdd pch w=2u l=180n
M2406 t930 nw269 vdd vdd pch w=2u l=180n
CT931 t931 0 0.1f
M2407 t930 nw268 t931 0 nch w=1u l=180n
M2408 t931 nw269 0 0 nch w=1u l=180n
M2409 nw274 t930 vdd vdd pch w=2u l=180n
M2410 nw274 t930 0 0 nch w=1u l=180n
Cnw274 nw274 0 2f
CT932 t932 0 0.1f
CT933 t933 0 0.1f
CT934 t934 0 0.1f
M2411 t932 na22 vdd vdd pch w=2u l=180n
M2412 t932 nb22 vdd vdd pch w=2u l=180n
CT935 t935 0 0.1f
M2413 t932 na22 t935 0 nch w=1u l=180n
M2414 t935 nb22 0 0 nch w=1u l=180n
M2415 t933 na22 vdd vdd pch w=2u l=180n
M2416 t933 t932 vdd vdd pch w=2u l=180n
CT936 t936 0 0.1f
M2417 t933 na22 t936 0 nch w=1u l=180n
M2418 t936 t932 0 0 nch w=1u l=180n
M2419 t934 nb22 vdd vdd pch w=2u l=180n
M2420 t934 t932 vdd vdd pch w=2u l=180n
CT937 t937 0 0.1f
M2421 t934 nb22 t937 0 nch w=1u l=180n
M2422 t937 t932 0 0 nch w=1u l=180n
CT938 t938 0 0.1f
M2423 t938 t933 vdd vdd pch w=2u l=180n
M2424 t938 t934 vdd vdd pch w=2u l=180n
CT939 t939 0 0.1f
M2425 t938 t933 t939 0 nch w=1u l=180n
M2426 t939 t934 0 0 nch w=1u l=180n
M2427 nw275 t938 vdd vdd pch w=2u l=180n
M2428 nw275 t938 0 0 nch w=1u l=180n
Cnw275 nw275 0 2f
M2429 nw276 nb22 vdd vdd pch w=2u l=180n
M2430 nw276 nb22 0 0 nch w=1u l=180n
Cnw276 nw276 0 2f
CT940 t940 0 0.1f
M2431 t940 na22 vdd vdd pch w=2u l=180n
M2432 t940 nw276 vdd vdd pch w=2u l=180n
CT941 t941 0 0.1f
M2433 t940 na22 t941 0 nch w=1u l=180n
M2434 t941 nw276 0 0 nch w=1u l=180n
M2435 nw277 t940 vdd vdd pch w=2u l=180n
M2436 nw277 t940 0 0 nch w=1u l=180n
Cnw277 nw277 0 2f
CT942 t942 0 0.1f
M2437 t942 nw274 vdd vdd pch w=2u l=180n
M2438 t942 nw277 vdd vdd pch w=2u l=180n
CT943 t943 0 0.1f
M2439 t942 nw274 t943 0 nch w=1u l=180n
M2440 t943 nw277 0 0 nch w=1u l=180n
M2441 nw278 t942 vdd vdd pch w=2u l=180n
M2442 nw278 t942 0 0 nch w=1u l=180n
Cnw278 nw278 0 2f
CT944 t944 0 0.1f
M2443 t944 nw273 0 0 nch w=1u l=180n
M2444 t944 nw278 0 0 nch w=1u l=180n
CT945 t945 0 0.1f
M2445 t945 nw273 vdd vdd pch w=2u l=180n
M2446 t944 nw278 t945 vdd pch w=2u l=180n
M2447 nw279 t944 vdd vdd pch w=2u l=180n
M2448 nw279 t944 0 0 nch w=1u l=180n
Cnw279 nw279 0 2f
CT946 t946 0 0.1f
M2449 t946 nw274 vdd vdd pch w=2u l=180n
M2450 t946 nw275 vdd vdd pch w=2u l=180n
CT947 t947 0 0.1f
M2451 t946 nw274 t947 0 nch w=1u l=180n
M2452 t947 nw275 0 0 nch w=1u l=180n
M2453 nw280 t946 vdd vdd pch w=2u l=180n
M2454 nw280 t946 0 0 nch w=1u l=180n
Cnw280 nw280 0 2f
CT948 t948 0 0.1f
CT949 t949 0 0.1f
CT950 t950 0 0.1f
M2455 t948 na21 vdd vdd pch w=2u l=180n
M2456 t948 nb21 vdd vdd pch w=2u l=180n
CT951 t951 0 0.1f
M2457 t948 na21 t951 0 nch w=1u l=180n
M2458 t951 nb21 0 0 nch w=1u l=180n
M2459 t949 na21 vdd vdd pch w=2u l=180n
M2460 t949 t948 vdd vdd pch w=2u l=180n
CT952 t952 0 0.1f
M2461 t949 na21 t952 0 nch w=1u l=180n
M2462 t952 t948 0 0 nch w=1u l=180n
M2463 t950 nb21 vdd vdd pch w=2u l=180n
M2464 t950 t948 vdd vdd pch w=2u l=180n
CT953 t953 0 0.1f
M2465 t950 nb21 t953 0 nch w=1u l=180n
M2466 t953 t948 0 0 nch w=1u l=180n
CT954 t954 0 0.1f
M2467 t954 t949 vdd vdd pch w=2u l=180n
M2468 t954 t950 vdd vdd pch w=2u l=180n
CT955 t955 0 0.1f
M2469 t954 t949 t955 0 nch w=1u l=180n
M2470 t955 t950 0 0 nch w=1u l=180n
M2471 nw281 t954 vdd vdd pch w=2u l=180n
M2472 nw281 t954 0 0 nch w=1u l=180n
Cnw281 nw281 0 2f
M2473 nw282 nb21 vdd vdd pch w=2u l=180n
M2474 nw282 nb21 0 0 nch w=1u l=180n
Cnw282 nw282 0 2f
CT956 t956 0 0.1f
M2475 t956 na21 vdd vdd pch w=2u l=180n
M2476 t956 nw282 vdd vdd pch w=2u l=180n
CT957 t957 0 0.1f
M2477 t956 na21 t957 0 nch w=1u l=180n
M2478 t957 nw282 0 0 nch w=1u l=180n
M2479 nw283 t956 vdd vdd pch w=2u l=180n
M2480 nw283 t956 0 0 nch w=1u l=180n
Cnw283 nw283 0 2f
CT958 t958 0 0.1f
M2481 t958 nw280 vdd vdd pch w=2u l=180n
M2482 t958 nw283 vdd vdd pch w=2u l=180n
CT959 t959 0 0.1f
M2483 t958 nw280 t959 0 nch w=1u l=180n
M2484 t959 nw283 0 0 nch w=1u l=180n
M2485 nw284 t958 vdd vdd pch w=2u l=180n
M2486 nw284 t958 0 0 nch w=1u l=180n
Cnw284 nw284 0 2f
CT960 t960 0 0.1f
M2487 t960 nw279 0 0 nch w=1u l=180n
M2488 t960 nw284 0 0 nch w=1u l=180n
CT961 t961 0 0.1f
M2489 t961 nw279 vdd vdd pch w=2u l=180n
M2490 t960 nw284 t961 vdd pch w=2u l=180n
M2491 nw285 t960 vdd vdd pch w=2u l=180n
M2492 nw285 t960 0 0 nch w=1u l=180n
Cnw285 nw285 0 2f
CT962 t962 0 0.1f
M2493 t962 nw280 vdd vdd pch w=2u l=180n
M2494 t962 nw281 vdd vdd pch w=2u l=180n
CT963 t963 0 0.1f
M2495 t962 nw280 t963 0 nch w=1u l=180n
M2496 t963 nw281 0 0 nch w=1u l=180n
M2497 nw286 t962 vdd vdd pch w=2u l=180n
M2498 nw286 t962 0 0 nch w=1u l=180n
Cnw286 nw286 0 2f
CT964 t964 0 0.1f
CT965 t965 0 0.1f
CT966 t966 0 0.1f
M2499 t964 na20 vdd vdd pch w=2u l=180n
M2500 t964 nb20 vdd vdd pch w=2u l=180n
CT967 t967 0 0.1f
M2501 t964 na20 t967 0 nch w=1u l=180n
M2502 t967 nb20 0 0 nch w=1u l=180n
M2503 t965 na20 vdd vdd pch w=2u l=180n
M2504 t965 t964 vdd vdd pch w=2u l=180n
CT968 t968 0 0.1f
M2505 t965 na20 t968 0 nch w=1u l=180n
M2506 t968 t964 0 0 nch w=1u l=180n
M2507 t966 nb20 vdd vdd pch w=2u l=180n
M2508 t966 t964 vdd vdd pch w=2u l=180n
CT969 t969 0 0.1f
M2509 t966 nb20 t969 0 nch w=1u l=180n
M2510 t969 t964 0 0 nch w=1u l=180n
CT970 t970 0 0.1f
M2511 t970 t965 vdd vdd pch w=2u l=180n
M2512 t970 t966 vdd vdd pch w=2u l=180n
CT971 t971 0 0.1f
M2513 t970 t965 t971 0 nch w=1u l=180n
M2514 t971 t966 0 0 nch w=1u l=180n
M2515 nw287 t970 vdd vdd pch w=2u l=180n
M2516 nw287 t970 0 0 nch w=1u l=180n
Cnw287 nw287 0 2f
M2517 nw288 nb20 vdd vdd pch w=2u l=180n
M2518 nw288 nb20 0 0 nch w=1u l=180n
Cnw288 nw288 0 2f
CT972 t972 0 0.1f
M2519 t972 na20 vdd vdd pch w=2u l=180n
M2520 t972 nw288 vdd vdd pch w=2u l=180n
CT973 t973 0 0.1f
M2521 t972 na20 t973 0 nch w=1u l=180n
M2522 t973 nw288 0 0 nch w=1u l=180n
M2523 nw289 t972 vdd vdd pch w=2u l=180n
M2524 nw289 t972 0 0 nch w=1u l=180n
Cnw289 nw289 0 2f
CT974 t974 0 0.1f
M2525 t974 nw286 vdd vdd pch w=2u l=180n
M2526 t974 nw289 vdd vdd pch w=2u l=180n
CT975 t975 0 0.1f
M2527 t974 nw286 t975 0 nch w=1u l=180n
M2528 t975 nw289 0 0 nch w=1u l=180n
M2529 nw290 t974 vdd vdd pch w=2u l=180n
M2530 nw290 t974 0 0 nch w=1u l=180n
Cnw290 nw290 0 2f
CT976 t976 0 0.1f
M2531 t976 nw285 0 0 nch w=1u l=180n
M2532 t976 nw290 0 0 nch w=1u l=180n
CT977 t977 0 0.1f
M2533 t977 nw285 vdd vdd pch w=2u l=180n
M2534 t976 nw290 t977 vdd pch w=2u l=180n
M2535 nw291 t976 vdd vdd pch w=2u l=180n
M2536 nw291 t976 0 0 nch w=1u l=180n
Cnw291 nw291 0 2f
CT978 t978 0 0.1f
M2537 t978 nw286 vdd vdd pch w=2u l=180n
M2538 t978 nw287 vdd vdd pch w=2u l=180n
CT979 t979 0 0.1f
M2539 t978 nw286 t979 0 nch w=1u l=180n
M2540 t979 nw287 0 0 nch w=1u l=180n
M2541 nw292 t978 vdd vdd pch w=2u l=180n
M2542 nw292 t978 0 0 nch w=1u l=180n
Cnw292 nw292 0 2f
CT980 t980 0 0.1f
CT981 t981 0 0.1f
CT982 t982 0 0.1f
M2543 t980 na19 vdd vdd pch w=2u l=180n
M2544 t980 nb19 vdd vdd pch w=2u l=180n
CT983 t983 0 0.1f
M2545 t980 na19 t983 0 nch w=1u l=180n
M2546 t983 nb19 0 0 nch w=1u l=180n
M2547 t981 na19 vdd vdd pch w=2u l=180n
M2548 t981 t980 vdd vdd pch w=2u l=180n
CT984 t984 0 0.1f
M2549 t981 na19 t984 0 nch w=1u l=180n
M2550 t984 t980 0 0 nch w=1u l=180n
M2551 t982 nb19 vdd vdd pch w=2u l=180n
M2552 t982 t980 vdd vdd pch w=2u l=180n
CT985 t985 0 0.1f
M2553 t982 nb19 t985 0 nch w=1u l=180n
M2554 t985 t980 0 0 nch w=1u l=180n
CT986 t986 0 0.1f
M2555 t986 t981 vdd vdd pch w=2u l=180n
M2556 t986 t982 vdd vdd pch w=2u l=180n
CT987 t987 0 0.1f
M2557 t986 t981 t987 0 nch w=1u l=180n
M2558 t987 t982 0 0 nch w=1u l=180n
M2559 nw293 t986 vdd vdd pch w=2u l=180n
M2560 nw293 t986 0 0 nch w=1u l=180n
Cnw293 nw293 0 2f
M2561 nw294 nb19 vdd vdd pch w=2u l=180n
M2562 nw294 nb19 0 0 nch w=1u l=180n
Cnw294 nw294 0 2f
CT988 t988 0 0.1f
M2563 t988 na19 vdd vdd pch w=2u l=180n
M2564 t988 nw294 vdd vdd pch w=2u l=180n
CT989 t989 0 0.1f
M2565 t988 na19 t989 0 nch w=1u l=180n
M2566 t989 nw294 0 0 nch w=1u l=180n
M2567 nw295 t988 vdd vdd pch w=2u l=180n
M2568 nw295 t988 0 0 nch w=1u l=180n
Cnw295 nw295 0 2f
CT990 t990 0 0.1f
M2569 t990 nw292 vdd vdd pch w=2u l=180n
M2570 t990 nw295 vdd vdd pch w=2u l=180n
CT991 t991 0 0.1f
M2571 t990 nw292 t991 0 nch w=1u l=180n
M2572 t991 nw295 0 0 nch w=1u l=180n
M2573 nw296 t990 vdd vdd pch w=2u l=180n
M2574 nw296 t990 0 0 nch w=1u l=180n
Cnw296 nw296 0 2f
CT992 t992 0 0.1f
M2575 t992 nw291 0 0 nch w=1u l=180n
M2576 t992 nw296 0 0 nch w=1u l=180n
CT993 t993 0 0.1f
M2577 t993 nw291 vdd vdd pch w=2u l=180n
M2578 t992 nw296 t993 vdd pch w=2u l=180n
M2579 nw297 t992 vdd vdd pch w=2u l=180n
M2580 nw297 t992 0 0 nch w=1u l=180n
Cnw297 nw297 0 2f
CT994 t994 0 0.1f
M2581 t994 nw292 vdd vdd pch w=2u l=180n
M2582 t994 nw293 vdd vdd pch w=2u l=180n
CT995 t995 0 0.1f
M2583 t994 nw292 t995 0 nch w=1u l=180n
M2584 t995 nw293 0 0 nch w=1u l=180n
M2585 nw298 t994 vdd vdd pch w=2u l=180n
M2586 nw298 t994 0 0 nch w=1u l=180n
Cnw298 nw298 0 2f
CT996 t996 0 0.1f
CT997 t997 0 0.1f
CT998 t998 0 0.1f
M2587 t996 na18 vdd vdd pch w=2u l=180n
M2588 t996 nb18 vdd vdd pch w=2u l=180n
CT999 t999 0 0.1f
M2589 t996 na18 t999 0 nch w=1u l=180n
M2590 t999 nb18 0 0 nch w=1u l=180n
M2591 t997 na18 vdd vdd pch w=2u l=180n
M2592 t997 t996 vdd vdd pch w=2u l=180n
CT1000 t1000 0 0.1f
M2593 t997 na18 t1000 0 nch w=1u l=180n
M2594 t1000 t996 0 0 nch w=1u l=180n
M2595 t998 nb18 vdd vdd pch w=2u l=180n
M2596 t998 t996 vdd vdd pch w=2u l=180n
CT1001 t1001 0 0.1f
M2597 t998 nb18 t1001 0 nch w=1u l=180n
M2598 t1001 t996 0 0 nch w=1u l=180n
CT1002 t1002 0 0.1f
M2599 t1002 t997 vdd vdd pch w=2u l=180n
M2600 t1002 t998 vdd vdd pch w=2u l=180n
CT1003 t1003 0 0.1f
M2601 t1002 t997 t1003 0 nch w=1u l=180n
M2602 t1003 t998 0 0 nch w=1u l=180n
M2603 nw299 t1002 vdd vdd pch w=2u l=180n
M2604 nw299 t1002 0 0 nch w=1u l=180n
Cnw299 nw299 0 2f
M2605 nw300 nb18 vdd vdd pch w=2u l=180n
M2606 nw300 nb18 0 0 nch w=1u l=180n
Cnw300 nw300 0 2f
CT1004 t1004 0 0.1f
M2607 t1004 na18 vdd vdd pch w=2u l=180n
M2608 t1004 nw300 vdd vdd pch w=2u l=180n
CT1005 t1005 0 0.1f
M2609 t1004 na18 t1005 0 nch w=1u l=180n
M2610 t1005 nw300 0 0 nch w=1u l=180n
M2611 nw301 t1004 vdd vdd pch w=2u l=180n
M2612 nw301 t1004 0 0 nch w=1u l=180n
Cnw301 nw301 0 2f
CT1006 t1006 0 0.1f
M2613 t1006 nw298 vdd vdd pch w=2u l=180n
M2614 t1006 nw301 vdd vdd pch w=2u l=180n
CT1007 t1007 0 0.1f
M2615 t1006 nw298 t1007 0 nch w=1u l=180n
M2616 t1007 nw301 0 0 nch w=1u l=180n
M2617 nw302 t1006 vdd vdd pch w=2u l=180n
M2618 nw302 t1006 0 0 nch w=1u l=180n
Cnw302 nw302 0 2f
CT1008 t1008 0 0.1f
M2619 t1008 nw297 0 0 nch w=1u l=180n
M2620 t1008 nw302 0 0 nch w=1u l=180n
CT1009 t1009 0 0.1f
M2621 t1009 nw297 vdd vdd pch w=2u l=180n
M2622 t1008 nw302 t1009 vdd pch w=2u l=180n
M2623 nw303 t1008 vdd vdd pch w=2u l=180n
M2624 nw303 t1008 0 0 nch w=1u l=180n
Cnw303 nw303 0 2f
CT1010 t1010 0 0.1f
M2625 t1010 nw298 vdd vdd pch w=2u l=180n
M2626 t1010 nw299 vdd vdd pch w=2u l=180n
CT1011 t1011 0 0.1f
M2627 t1010 nw298 t1011 0 nch w=1u l=180n
M2628 t1011 nw299 0 0 nch w=1u l=180n
M2629 nw304 t1010 vdd vdd pch w=2u l=180n
M2630 nw304 t1010 0 0 nch w=1u l=180n
Cnw304 nw304 0 2f
CT1012 t1012 0 0.1f
CT1013 t1013 0 0.1f
CT1014 t1014 0 0.1f
M2631 t1012 na17 vdd vdd pch w=2u l=180n
M2632 t1012 nb17 vdd vdd pch w=2u l=180n
CT1015 t1015 0 0.1f
M2633 t1012 na17 t1015 0 nch w=1u l=180n
M2634 t1015 nb17 0 0 nch w=1u l=180n
M2635 t1013 na17 vdd vdd pch w=2u l=180n
M2636 t1013 t1012 vdd vdd pch w=2u l=180n
CT1016 t1016 0 0.1f
M2637 t1013 na17 t1016 0 nch w=1u l=180n
M2638 t1016 t1012 0 0 nch w=1u l=180n
M2639 t1014 nb17 vdd vdd pch w=2u l=180n
M2640 t1014 t1012 vdd vdd pch w=2u l=180n
CT1017 t1017 0 0.1f
M2641 t1014 nb17 t1017 0 nch w=1u l=180n
M2642 t1017 t1012 0 0 nch w=1u l=180n
CT1018 t1018 0 0.1f
M2643 t1018 t1013 vdd vdd pch w=2u l=180n
M2644 t1018 t1014 vdd vdd pch w=2u l=180n
CT1019 t1019 0 0.1f
M2645 t1018 t1013 t1019 0 nch w=1u l=180n
M2646 t1019 t1014 0 0 nch w=1u l=180n
M2647 nw305 t1018 vdd vdd pch w=2u l=180n
M2648 nw305 t1018 0 0 nch w=1u l=180n
Cnw305 nw305 0 2f
M2649 nw306 nb17 vdd vdd pch w=2u l=180n
M2650 nw306 nb17 0 0 nch w=1u l=180n
Cnw306 nw306 0 2f
CT1020 t1020 0 0.1f
M2651 t1020 na17 vdd vdd pch w=2u l=180n
M2652 t1020 nw306 vdd vdd pch w=2u l=180n
CT1021 t1021 0 0.1f
M2653 t1020 na17 t1021 0 nch w=1u l=180n
M2654 t1021 nw306 0 0 nch w=1u l=180n
M2655 nw307 t1020 vdd vdd pch w=2u l=180n
M2656 nw307 t1020 0 0 nch w=1u l=180n
Cnw307 nw307 0 2f
CT1022 t1022 0 0.1f
M2657 t1022 nw304 vdd vdd pch w=2u l=180n
M2658 t1022 nw307 vdd vdd pch w=2u l=180n
CT1023 t1023 0 0.1f
M2659 t1022 nw304 t1023 0 nch w=1u l=180n
M2660 t1023 nw307 0 0 nch w=1u l=180n
M2661 nw308 t1022 vdd vdd pch w=2u l=180n
M2662 nw308 t1022 0 0 nch w=1u l=180n
Cnw308 nw308 0 2f
CT1024 t1024 0 0.1f
M2663 t1024 nw303 0 0 nch w=1u l=180n
M2664 t1024 nw308 0 0 nch w=1u l=180n
CT1025 t1025 0 0.1f
M2665 t1025 nw303 vdd vdd pch w=2u l=180n
M2666 t1024 nw308 t1025 vdd pch w=2u l=180n
M2667 nw309 t1024 vdd vdd pch w=2u l=180n
M2668 nw309 t1024 0 0 nch w=1u l=180n
Cnw309 nw309 0 2f
CT1026 t1026 0 0.1f
M2669 t1026 nw304 vdd vdd pch w=2u l=180n
M2670 t1026 nw305 vdd vdd pch w=2u l=180n
CT1027 t1027 0 0.1f
M2671 t1026 nw304 t1027 0 nch w=1u l=180n
M2672 t1027 nw305 0 0 nch w=1u l=180n
M2673 nw310 t1026 vdd vdd pch w=2u l=180n
M2674 nw310 t1026 0 0 nch w=1u l=180n
Cnw310 nw310 0 2f
CT1028 t1028 0 0.1f
CT1029 t1029 0 0.1f
CT1030 t1030 0 0.1f
M2675 t1028 na16 vdd vdd pch w=2u l=180n
M2676 t1028 nb16 vdd vdd pch w=2u l=180n
CT1031 t1031 0 0.1f
M2677 t1028 na16 t1031 0 nch w=1u l=180n
M2678 t1031 nb16 0 0 nch w=1u l=180n
M2679 t1029 na16 vdd vdd pch w=2u l=180n
M2680 t1029 t1028 vdd vdd pch w=2u l=180n
CT1032 t1032 0 0.1f
M2681 t1029 na16 t1032 0 nch w=1u l=180n
M2682 t1032 t1028 0 0 nch w=1u l=180n
M2683 t1030 nb16 vdd vdd pch w=2u l=180n
M2684 t1030 t1028 vdd vdd pch w=2u l=180n
CT1033 t1033 0 0.1f
M2685 t1030 nb16 t1033 0 nch w=1u l=180n
M2686 t1033 t1028 0 0 nch w=1u l=180n
CT1034 t1034 0 0.1f
M2687 t1034 t1029 vdd vdd pch w=2u l=180n
M2688 t1034 t1030 vdd vdd pch w=2u l=180n
CT1035 t1035 0 0.1f
M2689 t1034 t1029 t1035 0 nch w=1u l=180n
M2690 t1035 t1030 0 0 nch w=1u l=180n
M2691 nw311 t1034 vdd vdd pch w=2u l=180n
M2692 nw311 t1034 0 0 nch w=1u l=180n
Cnw311 nw311 0 2f
M2693 nw312 nb16 vdd vdd pch w=2u l=180n
M2694 nw312 nb16 0 0 nch w=1u l=180n
Cnw312 nw312 0 2f
CT1036 t1036 0 0.1f
M2695 t1036 na16 vdd vdd pch w=2u l=180n
M2696 t1036 nw312 vdd vdd pch w=2u l=180n
CT1037 t1037 0 0.1f
M2697 t1036 na16 t1037 0 nch w=1u l=180n
M2698 t1037 nw312 0 0 nch w=1u l=180n
M2699 nw313 t1036 vdd vdd pch w=2u l=180n
M2700 nw313 t1036 0 0 nch w=1u l=180n
Cnw313 nw313 0 2f
CT1038 t1038 0 0.1f
M2701 t1038 nw310 vdd vdd pch w=2u l=180n
M2702 t1038 nw313 vdd vdd pch w=2u l=180n
CT1039 t1039 0 0.1f
M2703 t1038 nw310 t1039 0 nch w=1u l=180n
M2704 t1039 nw313 0 0 nch w=1u l=180n
M2705 nw314 t1038 vdd vdd pch w=2u l=180n
M2706 nw314 t1038 0 0 nch w=1u l=180n
Cnw314 nw314 0 2f
CT1040 t1040 0 0.1f
M2707 t1040 nw309 0 0 nch w=1u l=180n
M2708 t1040 nw314 0 0 nch w=1u l=180n
CT1041 t1041 0 0.1f
M2709 t1041 nw309 vdd vdd pch w=2u l=180n
M2710 t1040 nw314 t1041 vdd pch w=2u l=180n
M2711 nw315 t1040 vdd vdd pch w=2u l=180n
M2712 nw315 t1040 0 0 nch w=1u l=180n
Cnw315 nw315 0 2f
CT1042 t1042 0 0.1f
M2713 t1042 nw310 vdd vdd pch w=2u l=180n
M2714 t1042 nw311 vdd vdd pch w=2u l=180n
CT1043 t1043 0 0.1f
M2715 t1042 nw310 t1043 0 nch w=1u l=180n
M2716 t1043 nw311 0 0 nch w=1u l=180n
M2717 nw316 t1042 vdd vdd pch w=2u l=180n
M2718 nw316 t1042 0 0 nch w=1u l=180n
Cnw316 nw316 0 2f
CT1044 t1044 0 0.1f
CT1045 t1045 0 0.1f
CT1046 t1046 0 0.1f
M2719 t1044 na15 vdd vdd pch w=2u l=180n
M2720 t1044 nb15 vdd vdd pch w=2u l=180n
CT1047 t1047 0 0.1f
M2721 t1044 na15 t1047 0 nch w=1u l=180n
M2722 t1047 nb15 0 0 nch w=1u l=180n
M2723 t1045 na15 vdd vdd pch w=2u l=180n
M2724 t1045 t1044 vdd vdd pch w=2u l=180n
CT1048 t1048 0 0.1f
M2725 t1045 na15 t1048 0 nch w=1u l=180n
M2726 t1048 t1044 0 0 nch w=1u l=180n
M2727 t1046 nb15 vdd vdd pch w=2u l=180n
M2728 t1046 t1044 vdd vdd pch w=2u l=180n
CT1049 t1049 0 0.1f
M2729 t1046 nb15 t1049 0 nch w=1u l=180n
M2730 t1049 t1044 0 0 nch w=1u l=180n
CT1050 t1050 0 0.1f
M2731 t1050 t1045 vdd vdd pch w=2u l=180n
M2732 t1050 t1046 vdd vdd pch w=2u l=180n
CT1051 t1051 0 0.1f
M2733 t1050 t1045 t1051 0 nch w=1u l=180n
M2734 t1051 t1046 0 0 nch w=1u l=180n
M2735 nw317 t1050 vdd vdd pch w=2u l=180n
M2736 nw317 t1050 0 0 nch w=1u l=180n
Cnw317 nw317 0 2f
M2737 nw318 nb15 vdd vdd pch w=2u l=180n
M2738 nw318 nb15 0 0 nch w=1u l=180n
Cnw318 nw318 0 2f
CT1052 t1052 0 0.1f
M2739 t1052 na15 vdd vdd pch w=2u l=180n
M2740 t1052 nw318 vdd vdd pch w=2u l=180n
CT1053 t1053 0 0.1f
M2741 t1052 na15 t1053 0 nch w=1u l=180n
M2742 t1053 nw318 0 0 nch w=1u l=180n
M2743 nw319 t1052 vdd vdd pch w=2u l=180n
M2744 nw319 t1052 0 0 nch w=1u l=180n
Cnw319 nw319 0 2f
CT1054 t1054 0 0.1f
M2745 t1054 nw316 vdd vdd pch w=2u l=180n
M2746 t1054 nw319 vdd vdd pch w=2u l=180n
CT1055 t1055 0 0.1f
M2747 t1054 nw316 t1055 0 nch w=1u l=180n
M2748 t1055 nw319 0 0 nch w=1u l=180n
M2749 nw320 t1054 vdd vdd pch w=2u l=180n
M2750 nw320 t1054 0 0 nch w=1u l=180n
Cnw320 nw320 0 2f
CT1056 t1056 0 0.1f
M2751 t1056 nw315 0 0 nch w=1u l=180n
M2752 t1056 nw320 0 0 nch w=1u l=180n
CT1057 t1057 0 0.1f
M2753 t1057 nw315 vdd vdd pch w=2u l=180n
M2754 t1056 nw320 t1057 vdd pch w=2u l=180n
M2755 nw321 t1056 vdd vdd pch w=2u l=180n
M2756 nw321 t1056 0 0 nch w=1u l=180n
Cnw321 nw321 0 2f
CT1058 t1058 0 0.1f
M2757 t1058 nw316 vdd vdd pch w=2u l=180n
M2758 t1058 nw317 vdd vdd pch w=2u l=180n
CT1059 t1059 0 0.1f
M2759 t1058 nw316 t1059 0 nch w=1u l=180n
M2760 t1059 nw317 0 0 nch w=1u l=180n
M2761 nw322 t1058 vdd vdd pch w=2u l=180n
M2762 nw322 t1058 0 0 nch w=1u l=180n
Cnw322 nw322 0 2f
CT1060 t1060 0 0.1f
CT1061 t1061 0 0.1f
CT1062 t1062 0 0.1f
M2763 t1060 na14 vdd vdd pch w=2u l=180n
M2764 t1060 nb14 vdd vdd pch w=2u l=180n
CT1063 t1063 0 0.1f
M2765 t1060 na14 t1063 0 nch w=1u l=180n
M2766 t1063 nb14 0 0 nch w=1u l=180n
M2767 t1061 na14 vdd vdd pch w=2u l=180n
M2768 t1061 t1060 vdd vdd pch w=2u l=180n
CT1064 t1064 0 0.1f
M2769 t1061 na14 t1064 0 nch w=1u l=180n
M2770 t1064 t1060 0 0 nch w=1u l=180n
M2771 t1062 nb14 vdd vdd pch w=2u l=180n
M2772 t1062 t1060 vdd vdd pch w=2u l=180n
CT1065 t1065 0 0.1f
M2773 t1062 nb14 t1065 0 nch w=1u l=180n
M2774 t1065 t1060 0 0 nch w=1u l=180n
CT1066 t1066 0 0.1f
M2775 t1066 t1061 vdd vdd pch w=2u l=180n
M2776 t1066 t1062 vdd vdd pch w=2u l=180n
CT1067 t1067 0 0.1f
M2777 t1066 t1061 t1067 0 nch w=1u l=180n
M2778 t1067 t1062 0 0 nch w=1u l=180n
M2779 nw323 t1066 vdd vdd pch w=2u l=180n
M2780 nw323 t1066 0 0 nch w=1u l=180n
Cnw323 nw323 0 2f
M2781 nw324 nb14 vdd vdd pch w=2u l=180n
M2782 nw324 nb14 0 0 nch w=1u l=180n
Cnw324 nw324 0 2f
CT1068 t1068 0 0.1f
M2783 t1068 na14 vdd vdd pch w=2u l=180n
M2784 t1068 nw324 vdd vdd pch w=2u l=180n
CT1069 t1069 0 0.1f
M2785 t1068 na14 t1069 0 nch w=1u l=180n
M2786 t1069 nw324 0 0 nch w=1u l=180n
M2787 nw325 t1068 vdd vdd pch w=2u l=180n
M2788 nw325 t1068 0 0 nch w=1u l=180n
Cnw325 nw325 0 2f
CT1070 t1070 0 0.1f
M2789 t1070 nw322 vdd vdd pch w=2u l=180n
M2790 t1070 nw325 vdd vdd pch w=2u l=180n
CT1071 t1071 0 0.1f
M2791 t1070 nw322 t1071 0 nch w=1u l=180n
M2792 t1071 nw325 0 0 nch w=1u l=180n
M2793 nw326 t1070 vdd vdd pch w=2u l=180n
M2794 nw326 t1070 0 0 nch w=1u l=180n
Cnw326 nw326 0 2f
CT1072 t1072 0 0.1f
M2795 t1072 nw321 0 0 nch w=1u l=180n
M2796 t1072 nw326 0 0 nch w=1u l=180n
CT1073 t1073 0 0.1f
M2797 t1073 nw321 vdd vdd pch w=2u l=180n
M2798 t1072 nw326 t1073 vdd pch w=2u l=180n
M2799 nw327 t1072 vdd vdd pch w=2u l=180n
M2800 nw327 t1072 0 0 nch w=1u l=180n
Cnw327 nw327 0 2f
CT1074 t1074 0 0.1f
M2801 t1074 nw322 vdd vdd pch w=2u l=180n
M2802 t1074 nw323 vdd vdd pch w=2u l=180n
CT1075 t1075 0 0.1f
M2803 t1074 nw322 t1075 0 nch w=1u l=180n
M2804 t1075 nw323 0 0 nch w=1u l=180n
M2805 nw328 t1074 vdd vdd pch w=2u l=180n
M2806 nw328 t1074 0 0 nch w=1u l=180n
Cnw328 nw328 0 2f
CT1076 t1076 0 0.1f
CT1077 t1077 0 0.1f
CT1078 t1078 0 0.1f
M2807 t1076 na13 vdd vdd pch w=2u l=180n
M2808 t1076 nb13 vdd vdd pch w=2u l=180n
CT1079 t1079 0 0.1f
M2809 t1076 na13 t1079 0 nch w=1u l=180n
M2810 t1079 nb13 0 0 nch w=1u l=180n
M2811 t1077 na13 vdd vdd pch w=2u l=180n
M2812 t1077 t1076 vdd vdd pch w=2u l=180n
CT1080 t1080 0 0.1f
M2813 t1077 na13 t1080 0 nch w=1u l=180n
M2814 t1080 t1076 0 0 nch w=1u l=180n
M2815 t1078 nb13 vdd vdd pch w=2u l=180n
M2816 t1078 t1076 vdd vdd pch w=2u l=180n
CT1081 t1081 0 0.1f
M2817 t1078 nb13 t1081 0 nch w=1u l=180n
M2818 t1081 t1076 0 0 nch w=1u l=180n
CT1082 t1082 0 0.1f
M2819 t1082 t1077 vdd vdd pch w=2u l=180n
M2820 t1082 t1078 vdd vdd pch w=2u l=180n
CT1083 t1083 0 0.1f
M2821 t1082 t1077 t1083 0 nch w=1u l=180n
M2822 t1083 t1078 0 0 nch w=1u l=180n
M2823 nw329 t1082 vdd vdd pch w=2u l=180n
M2824 nw329 t1082 0 0 nch w=1u l=180n
Cnw329 nw329 0 2f
M2825 nw330 nb13 vdd vdd pch w=2u l=180n
M2826 nw330 nb13 0 0 nch w=1u l=180n
Cnw330 nw330 0 2f
CT1084 t1084 0 0.1f
M2827 t1084 na13 vdd vdd pch w=2u l=180n
M2828 t1084 nw330 vdd vdd pch w=2u l=180n
CT1085 t1085 0 0.1f
M2829 t1084 na13 t1085 0 nch w=1u l=180n
M2830 t1085 nw330 0 0 nch w=1u l=180n
M2831 nw331 t1084 vdd vdd pch w=2u l=180n
M2832 nw331 t1084 0 0 nch w=1u l=180n
Cnw331 nw331 0 2f
CT1086 t1086 0 0.1f
M2833 t1086 nw328 vdd vdd pch w=2u l=180n
M2834 t1086 nw331 vdd vdd pch w=2u l=180n
CT1087 t1087 0 0.1f
M2835 t1086 nw328 t1087 0 nch w=1u l=180n
M2836 t1087 nw331 0 0 nch w=1u l=180n
M2837 nw332 t1086 vdd vdd pch w=2u l=180n
M2838 nw332 t1086 0 0 nch w=1u l=180n
Cnw332 nw332 0 2f
CT1088 t1088 0 0.1f
M2839 t1088 nw327 0 0 nch w=1u l=180n
M2840 t1088 nw332 0 0 nch w=1u l=180n
CT1089 t1089 0 0.1f
M2841 t1089 nw327 vdd vdd pch w=2u l=180n
M2842 t1088 nw332 t1089 vdd pch w=2u l=180n
M2843 nw333 t1088 vdd vdd pch w=2u l=180n
M2844 nw333 t1088 0 0 nch w=1u l=180n
Cnw333 nw333 0 2f
CT1090 t1090 0 0.1f
M2845 t1090 nw328 vdd vdd pch w=2u l=180n
M2846 t1090 nw329 vdd vdd pch w=2u l=180n
CT1091 t1091 0 0.1f
M2847 t1090 nw328 t1091 0 nch w=1u l=180n
M2848 t1091 nw329 0 0 nch w=1u l=180n
M2849 nw334 t1090 vdd vdd pch w=2u l=180n
M2850 nw334 t1090 0 0 nch w=1u l=180n
Cnw334 nw334 0 2f
CT1092 t1092 0 0.1f
CT1093 t1093 0 0.1f
CT1094 t1094 0 0.1f
M2851 t1092 na12 vdd vdd pch w=2u l=180n
M2852 t1092 nb12 vdd vdd pch w=2u l=180n
CT1095 t1095 0 0.1f
M2853 t1092 na12 t1095 0 nch w=1u l=180n
M2854 t1095 nb12 0 0 nch w=1u l=180n
M2855 t1093 na12 vdd vdd pch w=2u l=180n
M2856 t1093 t1092 vdd vdd pch w=2u l=180n
CT1096 t1096 0 0.1f
M2857 t1093 na12 t1096 0 nch w=1u l=180n
M2858 t1096 t1092 0 0 nch w=1u l=180n
M2859 t1094 nb12 vdd vdd pch w=2u l=180n
M2860 t1094 t1092 vdd vdd pch w=2u l=180n
CT1097 t1097 0 0.1f
M2861 t1094 nb12 t1097 0 nch w=1u l=180n
M2862 t1097 t1092 0 0 nch w=1u l=180n
CT1098 t1098 0 0.1f
M2863 t1098 t1093 vdd vdd pch w=2u l=180n
M2864 t1098 t1094 vdd vdd pch w=2u l=180n
CT1099 t1099 0 0.1f
M2865 t1098 t1093 t1099 0 nch w=1u l=180n
M2866 t1099 t1094 0 0 nch w=1u l=180n
M2867 nw335 t1098 vdd vdd pch w=2u l=180n
M2868 nw335 t1098 0 0 nch w=1u l=180n
Cnw335 nw335 0 2f
M2869 nw336 nb12 vdd vdd pch w=2u l=180n
M2870 nw336 nb12 0 0 nch w=1u l=180n
Cnw336 nw336 0 2f
CT1100 t1100 0 0.1f
M2871 t1100 na12 vdd vdd pch w=2u l=180n
M2872 t1100 nw336 vdd vdd pch w=2u l=180n
CT1101 t1101 0 0.1f
M2873 t1100 na12 t1101 0 nch w=1u l=180n
M2874 t1101 nw336 0 0 nch w=1u l=180n
M2875 nw337 t1100 vdd vdd pch w=2u l=180n
M2876 nw337 t1100 0 0 nch w=1u l=180n
Cnw337 nw337 0 2f
CT1102 t1102 0 0.1f
M2877 t1102 nw334 vdd vdd pch w=2u l=180n
M2878 t1102 nw337 vdd vdd pch w=2u l=180n
CT1103 t1103 0 0.1f
M2879 t1102 nw334 t1103 0 nch w=1u l=180n
M2880 t1103 nw337 0 0 nch w=1u l=180n
M2881 nw338 t1102 vdd vdd pch w=2u l=180n
M2882 nw338 t1102 0 0 nch w=1u l=180n
Cnw338 nw338 0 2f
CT1104 t1104 0 0.1f
M2883 t1104 nw333 0 0 nch w=1u l=180n
M2884 t1104 nw338 0 0 nch w=1u l=180n
CT1105 t1105 0 0.1f
M2885 t1105 nw333 vdd vdd pch w=2u l=180n
M2886 t1104 nw338 t1105 vdd pch w=2u l=180n
M2887 nw339 t1104 vdd vdd pch w=2u l=180n
M2888 nw339 t1104 0 0 nch w=1u l=180n
Cnw339 nw339 0 2f
CT1106 t1106 0 0.1f
M2889 t1106 nw334 vdd vdd pch w=2u l=180n
M2890 t1106 nw335 vdd vdd pch w=2u l=180n
CT1107 t1107 0 0.1f
M2891 t1106 nw334 t1107 0 nch w=1u l=180n
M2892 t1107 nw335 0 0 nch w=1u l=180n
M2893 nw340 t1106 vdd vdd pch w=2u l=180n
M2894 nw340 t1106 0 0 nch w=1u l=180n
Cnw340 nw340 0 2f
CT1108 t1108 0 0.1f
CT1109 t1109 0 0.1f
CT1110 t1110 0 0.1f
M2895 t1108 na11 vdd vdd pch w=2u l=180n
M2896 t1108 nb11 vdd vdd pch w=2u l=180n
CT1111 t1111 0 0.1f
M2897 t1108 na11 t1111 0 nch w=1u l=180n
M2898 t1111 nb11 0 0 nch w=1u l=180n
M2899 t1109 na11 vdd vdd pch w=2u l=180n
M2900 t1109 t1108 vdd vdd pch w=2u l=180n
CT1112 t1112 0 0.1f
M2901 t1109 na11 t1112 0 nch w=1u l=180n
M2902 t1112 t1108 0 0 nch w=1u l=180n
M2903 t1110 nb11 vdd vdd pch w=2u l=180n
M2904 t1110 t1108 vdd vdd pch w=2u l=180n
CT1113 t1113 0 0.1f
M2905 t1110 nb11 t1113 0 nch w=1u l=180n
M2906 t1113 t1108 0 0 nch w=1u l=180n
CT1114 t1114 0 0.1f
M2907 t1114 t1109 vdd vdd pch w=2u l=180n
M2908 t1114 t1110 vdd vdd pch w=2u l=180n
CT1115 t1115 0 0.1f
M2909 t1114 t1109 t1115 0 nch w=1u l=180n
M2910 t1115 t1110 0 0 nch w=1u l=180n
M2911 nw341 t1114 vdd vdd pch w=2u l=180n
M2912 nw341 t1114 0 0 nch w=1u l=180n
Cnw341 nw341 0 2f
M2913 nw342 nb11 vdd vdd pch w=2u l=180n
M2914 nw342 nb11 0 0 nch w=1u l=180n
Cnw342 nw342 0 2f
CT1116 t1116 0 0.1f
M2915 t1116 na11 vdd vdd pch w=2u l=180n
M2916 t1116 nw342 vdd vdd pch w=2u l=180n
CT1117 t1117 0 0.1f
M2917 t1116 na11 t1117 0 nch w=1u l=180n
M2918 t1117 nw342 0 0 nch w=1u l=180n
M2919 nw343 t1116 vdd vdd pch w=2u l=180n
M2920 nw343 t1116 0 0 nch w=1u l=180n
Cnw343 nw343 0 2f
CT1118 t1118 0 0.1f
M2921 t1118 nw340 vdd vdd pch w=2u l=180n
M2922 t1118 nw343 vdd vdd pch w=2u l=180n
CT1119 t1119 0 0.1f
M2923 t1118 nw340 t1119 0 nch w=1u l=180n
M2924 t1119 nw343 0 0 nch w=1u l=180n
M2925 nw344 t1118 vdd vdd pch w=2u l=180n
M2926 nw344 t1118 0 0 nch w=1u l=180n
Cnw344 nw344 0 2f
CT1120 t1120 0 0.1f
M2927 t1120 nw339 0 0 nch w=1u l=180n
M2928 t1120 nw344 0 0 nch w=1u l=180n
CT1121 t1121 0 0.1f
M2929 t1121 nw339 vdd vdd pch w=2u l=180n
M2930 t1120 nw344 t1121 vdd pch w=2u l=180n
M2931 nw345 t1120 vdd vdd pch w=2u l=180n
M2932 nw345 t1120 0 0 nch w=1u l=180n
Cnw345 nw345 0 2f
CT1122 t1122 0 0.1f
M2933 t1122 nw340 vdd vdd pch w=2u l=180n
M2934 t1122 nw341 vdd vdd pch w=2u l=180n
CT1123 t1123 0 0.1f
M2935 t1122 nw340 t1123 0 nch w=1u l=180n
M2936 t1123 nw341 0 0 nch w=1u l=180n
M2937 nw346 t1122 vdd vdd pch w=2u l=180n
M2938 nw346 t1122 0 0 nch w=1u l=180n
Cnw346 nw346 0 2f
CT1124 t1124 0 0.1f
CT1125 t1125 0 0.1f
CT1126 t1126 0 0.1f
M2939 t1124 na10 vdd vdd pch w=2u l=180n
M2940 t1124 nb10 vdd vdd pch w=2u l=180n
CT1127 t1127 0 0.1f
M2941 t1124 na10 t1127 0 nch w=1u l=180n
M2942 t1127 nb10 0 0 nch w=1u l=180n
M2943 t1125 na10 vdd vdd pch w=2u l=180n
M2944 t1125 t1124 vdd vdd pch w=2u l=180n
CT1128 t1128 0 0.1f
M2945 t1125 na10 t1128 0 nch w=1u l=180n
M2946 t1128 t1124 0 0 nch w=1u l=180n
M2947 t1126 nb10 vdd vdd pch w=2u l=180n
M2948 t1126 t1124 vdd vdd pch w=2u l=180n
CT1129 t1129 0 0.1f
M2949 t1126 nb10 t1129 0 nch w=1u l=180n
M2950 t1129 t1124 0 0 nch w=1u l=180n
CT1130 t1130 0 0.1f
M2951 t1130 t1125 vdd vdd pch w=2u l=180n
M2952 t1130 t1126 vdd vdd pch w=2u l=180n
CT1131 t1131 0 0.1f
M2953 t1130 t1125 t1131 0 nch w=1u l=180n
M2954 t1131 t1126 0 0 nch w=1u l=180n
M2955 nw347 t1130 vdd vdd pch w=2u l=180n
M2956 nw347 t1130 0 0 nch w=1u l=180n
Cnw347 nw347 0 2f
M2957 nw348 nb10 vdd vdd pch w=2u l=180n
M2958 nw348 nb10 0 0 nch w=1u l=180n
Cnw348 nw348 0 2f
CT1132 t1132 0 0.1f
M2959 t1132 na10 vdd vdd pch w=2u l=180n
M2960 t1132 nw348 vdd vdd pch w=2u l=180n
CT1133 t1133 0 0.1f
M2961 t1132 na10 t1133 0 nch w=1u l=180n
M2962 t1133 nw348 0 0 nch w=1u l=180n
M2963 nw349 t1132 vdd vdd pch w=2u l=180n
M2964 nw349 t1132 0 0 nch w=1u l=180n
Cnw349 nw349 0 2f
CT1134 t1134 0 0.1f
M2965 t1134 nw346 vdd vdd pch w=2u l=180n
M2966 t1134 nw349 vdd vdd pch w=2u l=180n
CT1135 t1135 0 0.1f
M2967 t1134 nw346 t1135 0 nch w=1u l=180n
M2968 t1135 nw349 0 0 nch w=1u l=180n
M2969 nw350 t1134 vdd vdd pch w=2u l=180n
M2970 nw350 t1134 0 0 nch w=1u l=180n
Cnw350 nw350 0 2f
CT1136 t1136 0 0.1f
M2971 t1136 nw345 0 0 nch w=1u l=180n
M2972 t1136 nw350 0 0 nch w=1u l=180n
CT1137 t1137 0 0.1f
M2973 t1137 nw345 vdd vdd pch w=2u l=180n
M2974 t1136 nw350 t1137 vdd pch w=2u l=180n
M2975 nw351 t1136 vdd vdd pch w=2u l=180n
M2976 nw351 t1136 0 0 nch w=1u l=180n
Cnw351 nw351 0 2f
CT1138 t1138 0 0.1f
M2977 t1138 nw346 vdd vdd pch w=2u l=180n
M2978 t1138 nw347 vdd vdd pch w=2u l=180n
CT1139 t1139 0 0.1f
M2979 t1138 nw346 t1139 0 nch w=1u l=180n
M2980 t1139 nw347 0 0 nch w=1u l=180n
M2981 nw352 t1138 vdd vdd pch w=2u l=180n
M2982 nw352 t1138 0 0 nch w=1u l=180n
Cnw352 nw352 0 2f
CT1140 t1140 0 0.1f
CT1141 t1141 0 0.1f
CT1142 t1142 0 0.1f
M2983 t1140 na9 vdd vdd pch w=2u l=180n
M2984 t1140 nb9 vdd vdd pch w=2u l=180n
CT1143 t1143 0 0.1f
M2985 t1140 na9 t1143 0 nch w=1u l=180n
M2986 t1143 nb9 0 0 nch w=1u l=180n
M2987 t1141 na9 vdd vdd pch w=2u l=180n
M2988 t1141 t1140 vdd vdd pch w=2u l=180n
CT1144 t1144 0 0.1f
M2989 t1141 na9 t1144 0 nch w=1u l=180n
M2990 t1144 t1140 0 0 nch w=1u l=180n
M2991 t1142 nb9 vdd vdd pch w=2u l=180n
M2992 t1142 t1140 vdd vdd pch w=2u l=180n
CT1145 t1145 0 0.1f
M2993 t1142 nb9 t1145 0 nch w=1u l=180n
M2994 t1145 t1140 0 0 nch w=1u l=180n
CT1146 t1146 0 0.1f
M2995 t1146 t1141 vdd vdd pch w=2u l=180n
M2996 t1146 t1142 vdd vdd pch w=2u l=180n
CT1147 t1147 0 0.1f
M2997 t1146 t1141 t1147 0 nch w=1u l=180n
M2998 t1147 t1142 0 0 nch w=1u l=180n
M2999 nw353 t1146 vdd vdd pch w=2u l=180n
M3000 nw353 t1146 0 0 nch w=1u l=180n
Cnw353 nw353 0 2f
M3001 nw354 nb9 vdd vdd pch w=2u l=180n
M3002 nw354 nb9 0 0 nch w=1u l=180n
Cnw354 nw354 0 2f
CT1148 t1148 0 0.1f
M3003 t1148 na9 vdd vdd pch w=2u l=180n
M3004 t1148 nw354 vdd vdd pch w=2u l=180n
CT1149 t1149 0 0.1f
M3005 t1148 na9 t1149 0 nch w=1u l=180n
M3006 t1149 nw354 0 0 nch w=1u l=180n
M3007 nw355 t1148 vdd vdd pch w=2u l=180n
M3008 nw355 t1148 0 0 nch w=1u l=180n
Cnw355 nw355 0 2f
CT1150 t1150 0 0.1f
M3009 t1150 nw352 vdd vdd pch w=2u l=180n
M3010 t1150 nw355 vdd vdd pch w=2u l=180n
CT1151 t1151 0 0.1f
M3011 t1150 nw352 t1151 0 nch w=1u l=180n
M3012 t1151 nw355 0 0 nch w=1u l=180n
M3013 nw356 t1150 vdd vdd pch w=2u l=180n
M3014 nw356 t1150 0 0 nch w=1u l=180n
Cnw356 nw356 0 2f
CT1152 t1152 0 0.1f
M3015 t1152 nw351 0 0 nch w=1u l=180n
M3016 t1152 nw356 0 0 nch w=1u l=180n
CT1153 t1153 0 0.1f
M3017 t1153 nw351 vdd vdd pch w=2u l=180n
M3018 t1152 nw356 t1153 vdd pch w=2u l=180n
M3019 nw357 t1152 vdd vdd pch w=2u l=180n
M3020 nw357 t1152 0 0 nch w=1u l=180n
Cnw357 nw357 0 2f
CT1154 t1154 0 0.1f
M3021 t1154 nw352 vdd vdd pch w=2u l=180n
M3022 t1154 nw353 vdd vdd pch w=2u l=180n
CT1155 t1155 0 0.1f
M3023 t1154 nw352 t1155 0 nch w=1u l=180n
M3024 t1155 nw353 0 0 nch w=1u l=180n
M3025 nw358 t1154 vdd vdd pch w=2u l=180n
M3026 nw358 t1154 0 0 nch w=1u l=180n
Cnw358 nw358 0 2f
CT1156 t1156 0 0.1f
CT1157 t1157 0 0.1f
CT1158 t1158 0 0.1f
M3027 t1156 na8 vdd vdd pch w=2u l=180n
M3028 t1156 nb8 vdd vdd pch w=2u l=180n
CT1159 t1159 0 0.1f
M3029 t1156 na8 t1159 0 nch w=1u l=180n
M3030 t1159 nb8 0 0 nch w=1u l=180n
M3031 t1157 na8 vdd vdd pch w=2u l=180n
M3032 t1157 t1156 vdd vdd pch w=2u l=180n
CT1160 t1160 0 0.1f
M3033 t1157 na8 t1160 0 nch w=1u l=180n
M3034 t1160 t1156 0 0 nch w=1u l=180n
M3035 t1158 nb8 vdd vdd pch w=2u l=180n
M3036 t1158 t1156 vdd vdd pch w=2u l=180n
CT1161 t1161 0 0.1f
M3037 t1158 nb8 t1161 0 nch w=1u l=180n
M3038 t1161 t1156 0 0 nch w=1u l=180n
CT1162 t1162 0 0.1f
M3039 t1162 t1157 vdd vdd pch w=2u l=180n
M3040 t1162 t1158 vdd vdd pch w=2u l=180n
CT1163 t1163 0 0.1f
M3041 t1162 t1157 t1163 0 nch w=1u l=180n
M3042 t1163 t1158 0 0 nch w=1u l=180n
M3043 nw359 t1162 vdd vdd pch w=2u l=180n
M3044 nw359 t1162 0 0 nch w=1u l=180n
Cnw359 nw359 0 2f
M3045 nw360 nb8 vdd vdd pch w=2u l=180n
M3046 nw360 nb8 0 0 nch w=1u l=180n
Cnw360 nw360 0 2f
CT1164 t1164 0 0.1f
M3047 t1164 na8 vdd vdd pch w=2u l=180n
M3048 t1164 nw360 vdd vdd pch w=2u l=180n
CT1165 t1165 0 0.1f
M3049 t1164 na8 t1165 0 nch w=1u l=180n
M3050 t1165 nw360 0 0 nch w=1u l=180n
M3051 nw361 t1164 vdd vdd pch w=2u l=180n
M3052 nw361 t1164 0 0 nch w=1u l=180n
Cnw361 nw361 0 2f
CT1166 t1166 0 0.1f
M3053 t1166 nw358 vdd vdd pch w=2u l=180n
M3054 t1166 nw361 vdd vdd pch w=2u l=180n
CT1167 t1167 0 0.1f
M3055 t1166 nw358 t1167 0 nch w=1u l=180n
M3056 t1167 nw361 0 0 nch w=1u l=180n
M3057 nw362 t1166 vdd vdd pch w=2u l=180n
M3058 nw362 t1166 0 0 nch w=1u l=180n
Cnw362 nw362 0 2f
CT1168 t1168 0 0.1f
M3059 t1168 nw357 0 0 nch w=1u l=180n
M3060 t1168 nw362 0 0 nch w=1u l=180n
CT1169 t1169 0 0.1f
M3061 t1169 nw357 vdd vdd pch w=2u l=180n
M3062 t1168 nw362 t1169 vdd pch w=2u l=180n
M3063 nw363 t1168 vdd vdd pch w=2u l=180n
M3064 nw363 t1168 0 0 nch w=1u l=180n
Cnw363 nw363 0 2f
CT1170 t1170 0 0.1f
M3065 t1170 nw358 vdd vdd pch w=2u l=180n
M3066 t1170 nw359 vdd vdd pch w=2u l=180n
CT1171 t1171 0 0.1f
M3067 t1170 nw358 t1171 0 nch w=1u l=180n
M3068 t1171 nw359 0 0 nch w=1u l=180n
M3069 nw364 t1170 vdd vdd pch w=2u l=180n
M3070 nw364 t1170 0 0 nch w=1u l=180n
Cnw364 nw364 0 2f
CT1172 t1172 0 0.1f
CT1173 t1173 0 0.1f
CT1174 t1174 0 0.1f
M3071 t1172 na7 vdd vdd pch w=2u l=180n
M3072 t1172 nb7 vdd vdd pch w=2u l=180n
CT1175 t1175 0 0.1f
M3073 t1172 na7 t1175 0 nch w=1u l=180n
M3074 t1175 nb7 0 0 nch w=1u l=180n
M3075 t1173 na7 vdd vdd pch w=2u l=180n
M3076 t1173 t1172 vdd vdd pch w=2u l=180n
CT1176 t1176 0 0.1f
M3077 t1173 na7 t1176 0 nch w=1u l=180n
M3078 t1176 t1172 0 0 nch w=1u l=180n
M3079 t1174 nb7 vdd vdd pch w=2u l=180n
M3080 t1174 t1172 vdd vdd pch w=2u l=180n
CT1177 t1177 0 0.1f
M3081 t1174 nb7 t1177 0 nch w=1u l=180n
M3082 t1177 t1172 0 0 nch w=1u l=180n
CT1178 t1178 0 0.1f
M3083 t1178 t1173 vdd vdd pch w=2u l=180n
M3084 t1178 t1174 vdd vdd pch w=2u l=180n
CT1179 t1179 0 0.1f
M3085 t1178 t1173 t1179 0 nch w=1u l=180n
M3086 t1179 t1174 0 0 nch w=1u l=180n
M3087 nw365 t1178 vdd vdd pch w=2u l=180n
M3088 nw365 t1178 0 0 nch w=1u l=180n
Cnw365 nw365 0 2f
M3089 nw366 nb7 vdd vdd pch w=2u l=180n
M3090 nw366 nb7 0 0 nch w=1u l=180n
Cnw366 nw366 0 2f
CT1180 t1180 0 0.1f
M3091 t1180 na7 vdd vdd pch w=2u l=180n
M3092 t1180 nw366 vdd vdd pch w=2u l=180n
CT1181 t1181 0 0.1f
M3093 t1180 na7 t1181 0 nch w=1u l=180n
M3094 t1181 nw366 0 0 nch w=1u l=180n
M3095 nw367 t1180 vdd vdd pch w=2u l=180n
M3096 nw367 t1180 0 0 nch w=1u l=180n
Cnw367 nw367 0 2f
CT1182 t1182 0 0.1f
M3097 t1182 nw364 vdd vdd pch w=2u l=180n
M3098 t1182 nw367 vdd vdd pch w=2u l=180n
CT1183 t1183 0 0.1f
M3099 t1182 nw364 t1183 0 nch w=1u l=180n
M3100 t1183 nw367 0 0 nch w=1u l=180n
M3101 nw368 t1182 vdd vdd pch w=2u l=180n
M3102 nw368 t1182 0 0 nch w=1u l=180n
Cnw368 nw368 0 2f
CT1184 t1184 0 0.1f
M3103 t1184 nw363 0 0 nch w=1u l=180n
M3104 t1184 nw368 0 0 nch w=1u l=180n
CT1185 t1185 0 0.1f
M3105 t1185 nw363 vdd vdd pch w=2u l=180n
M3106 t1184 nw368 t1185 vdd pch w=2u l=180n
M3107 nw369 t1184 vdd vdd pch w=2u l=180n
M3108 nw369 t1184 0 0 nch w=1u l=180n
Cnw369 nw369 0 2f
CT1186 t1186 0 0.1f
M3109 t1186 nw364 vdd vdd pch w=2u l=180n
M3110 t1186 nw365 vdd vdd pch w=2u l=180n
CT1187 t1187 0 0.1f
M3111 t1186 nw364 t1187 0 nch w=1u l=180n
M3112 t1187 nw365 0 0 nch w=1u l=180n
M3113 nw370 t1186 vdd vdd pch w=2u l=180n
M3114 nw370 t1186 0 0 nch w=1u l=180n
Cnw370 nw370 0 2f
CT1188 t1188 0 0.1f
CT1189 t1189 0 0.1f
CT1190 t1190 0 0.1f
M3115 t1188 na6 vdd vdd pch w=2u l=180n
M3116 t1188 nb6 vdd vdd pch w=2u l=180n
CT1191 t1191 0 0.1f
M3117 t1188 na6 t1191 0 nch w=1u l=180n
M3118 t1191 nb6 0 0 nch w=1u l=180n
M3119 t1189 na6 vdd vdd pch w=2u l=180n
M3120 t1189 t1188 vdd vdd pch w=2u l=180n
CT1192 t1192 0 0.1f
M3121 t1189 na6 t1192 0 nch w=1u l=180n
M3122 t1192 t1188 0 0 nch w=1u l=180n
M3123 t1190 nb6 vdd vdd pch w=2u l=180n
M3124 t1190 t1188 vdd vdd pch w=2u l=180n
CT1193 t1193 0 0.1f
M3125 t1190 nb6 t1193 0 nch w=1u l=180n
M3126 t1193 t1188 0 0 nch w=1u l=180n
CT1194 t1194 0 0.1f
M3127 t1194 t1189 vdd vdd pch w=2u l=180n
M3128 t1194 t1190 vdd vdd pch w=2u l=180n
CT1195 t1195 0 0.1f
M3129 t1194 t1189 t1195 0 nch w=1u l=180n
M3130 t1195 t1190 0 0 nch w=1u l=180n
M3131 nw371 t1194 vdd vdd pch w=2u l=180n
M3132 nw371 t1194 0 0 nch w=1u l=180n
Cnw371 nw371 0 2f
M3133 nw372 nb6 vdd vdd pch w=2u l=180n
M3134 nw372 nb6 0 0 nch w=1u l=180n
Cnw372 nw372 0 2f
CT1196 t1196 0 0.1f
M3135 t1196 na6 vdd vdd pch w=2u l=180n
M3136 t1196 nw372 vdd vdd pch w=2u l=180n
CT1197 t1197 0 0.1f
M3137 t1196 na6 t1197 0 nch w=1u l=180n
M3138 t1197 nw372 0 0 nch w=1u l=180n
M3139 nw373 t1196 vdd vdd pch w=2u l=180n
M3140 nw373 t1196 0 0 nch w=1u l=180n
Cnw373 nw373 0 2f
CT1198 t1198 0 0.1f
M3141 t1198 nw370 vdd vdd pch w=2u l=180n
M3142 t1198 nw373 vdd vdd pch w=2u l=180n
CT1199 t1199 0 0.1f
M3143 t1198 nw370 t1199 0 nch w=1u l=180n
M3144 t1199 nw373 0 0 nch w=1u l=180n
M3145 nw374 t1198 vdd vdd pch w=2u l=180n
M3146 nw374 t1198 0 0 nch w=1u l=180n
Cnw374 nw374 0 2f
CT1200 t1200 0 0.1f
M3147 t1200 nw369 0 0 nch w=1u l=180n
M3148 t1200 nw374 0 0 nch w=1u l=180n
CT1201 t1201 0 0.1f
M3149 t1201 nw369 vdd vdd pch w=2u l=180n
M3150 t1200 nw374 t1201 vdd pch w=2u l=180n
M3151 nw375 t1200 vdd vdd pch w=2u l=180n
M3152 nw375 t1200 0 0 nch w=1u l=180n
Cnw375 nw375 0 2f
CT1202 t1202 0 0.1f
M3153 t1202 nw370 vdd vdd pch w=2u l=180n
M3154 t1202 nw371 vdd vdd pch w=2u l=180n
CT1203 t1203 0 0.1f
M3155 t1202 nw370 t1203 0 nch w=1u l=180n
M3156 t1203 nw371 0 0 nch w=1u l=180n
M3157 nw376 t1202 vdd vdd pch w=2u l=180n
M3158 nw376 t1202 0 0 nch w=1u l=180n
Cnw376 nw376 0 2f
CT1204 t1204 0 0.1f
CT1205 t1205 0 0.1f
CT1206 t1206 0 0.1f
M3159 t1204 na5 vdd vdd pch w=2u l=180n
M3160 t1204 nb5 vdd vdd pch w=2u l=180n
CT1207 t1207 0 0.1f
M3161 t1204 na5 t1207 0 nch w=1u l=180n
M3162 t1207 nb5 0 0 nch w=1u l=180n
M3163 t1205 na5 vdd vdd pch w=2u l=180n
M3164 t1205 t1204 vdd vdd pch w=2u l=180n
CT1208 t1208 0 0.1f
M3165 t1205 na5 t1208 0 nch w=1u l=180n
M3166 t1208 t1204 0 0 nch w=1u l=180n
M3167 t1206 nb5 vdd vdd pch w=2u l=180n
M3168 t1206 t1204 vdd vdd pch w=2u l=180n
CT1209 t1209 0 0.1f
M3169 t1206 nb5 t1209 0 nch w=1u l=180n
M3170 t1209 t1204 0 0 nch w=1u l=180n
CT1210 t1210 0 0.1f
M3171 t1210 t1205 vdd vdd pch w=2u l=180n
M3172 t1210 t1206 vdd vdd pch w=2u l=180n
CT1211 t1211 0 0.1f
M3173 t1210 t1205 t1211 0 nch w=1u l=180n
M3174 t1211 t1206 0 0 nch w=1u l=180n
M3175 nw377 t1210 vdd vdd pch w=2u l=180n
M3176 nw377 t1210 0 0 nch w=1u l=180n
Cnw377 nw377 0 2f
M3177 nw378 nb5 vdd vdd pch w=2u l=180n
M3178 nw378 nb5 0 0 nch w=1u l=180n
Cnw378 nw378 0 2f
CT1212 t1212 0 0.1f
M3179 t1212 na5 vdd vdd pch w=2u l=180n
M3180 t1212 nw378 vdd vdd pch w=2u l=180n
CT1213 t1213 0 0.1f
M3181 t1212 na5 t1213 0 nch w=1u l=180n
M3182 t1213 nw378 0 0 nch w=1u l=180n
M3183 nw379 t1212 vdd vdd pch w=2u l=180n
M3184 nw379 t1212 0 0 nch w=1u l=180n
Cnw379 nw379 0 2f
CT1214 t1214 0 0.1f
M3185 t1214 nw376 vdd vdd pch w=2u l=180n
M3186 t1214 nw379 vdd vdd pch w=2u l=180n
CT1215 t1215 0 0.1f
M3187 t1214 nw376 t1215 0 nch w=1u l=180n
M3188 t1215 nw379 0 0 nch w=1u l=180n
M3189 nw380 t1214 vdd vdd pch w=2u l=180n
M3190 nw380 t1214 0 0 nch w=1u l=180n
Cnw380 nw380 0 2f
CT1216 t1216 0 0.1f
M3191 t1216 nw375 0 0 nch w=1u l=180n
M3192 t1216 nw380 0 0 nch w=1u l=180n
CT1217 t1217 0 0.1f
M3193 t1217 nw375 vdd vdd pch w=2u l=180n
M3194 t1216 nw380 t1217 vdd pch w=2u l=180n
M3195 nw381 t1216 vdd vdd pch w=2u l=180n
M3196 nw381 t1216 0 0 nch w=1u l=180n
Cnw381 nw381 0 2f
CT1218 t1218 0 0.1f
M3197 t1218 nw376 vdd vdd pch w=2u l=180n
M3198 t1218 nw377 vdd vdd pch w=2u l=180n
CT1219 t1219 0 0.1f
M3199 t1218 nw376 t1219 0 nch w=1u l=180n
M3200 t1219 nw377 0 0 nch w=1u l=180n
M3201 nw382 t1218 vdd vdd pch w=2u l=180n
M3202 nw382 t1218 0 0 nch w=1u l=180n
Cnw382 nw382 0 2f
CT1220 t1220 0 0.1f
CT1221 t1221 0 0.1f
CT1222 t1222 0 0.1f
M3203 t1220 na4 vdd vdd pch w=2u l=180n
M3204 t1220 nb4 vdd vdd pch w=2u l=180n
CT1223 t1223 0 0.1f
M3205 t1220 na4 t1223 0 nch w=1u l=180n
M3206 t1223 nb4 0 0 nch w=1u l=180n
M3207 t1221 na4 vdd vdd pch w=2u l=180n
M3208 t1221 t1220 vdd vdd pch w=2u l=180n
CT1224 t1224 0 0.1f
M3209 t1221 na4 t1224 0 nch w=1u l=180n
M3210 t1224 t1220 0 0 nch w=1u l=180n
M3211 t1222 nb4 vdd vdd pch w=2u l=180n
M3212 t1222 t1220 vdd vdd pch w=2u l=180n
CT1225 t1225 0 0.1f
M3213 t1222 nb4 t1225 0 nch w=1u l=180n
M3214 t1225 t1220 0 0 nch w=1u l=180n
CT1226 t1226 0 0.1f
M3215 t1226 t1221 vdd vdd pch w=2u l=180n
M3216 t1226 t1222 vdd vdd pch w=2u l=180n
CT1227 t1227 0 0.1f
M3217 t1226 t1221 t1227 0 nch w=1u l=180n
M3218 t1227 t1222 0 0 nch w=1u l=180n
M3219 nw383 t1226 vdd vdd pch w=2u l=180n
M3220 nw383 t1226 0 0 nch w=1u l=180n
Cnw383 nw383 0 2f
M3221 nw384 nb4 vdd vdd pch w=2u l=180n
M3222 nw384 nb4 0 0 nch w=1u l=180n
Cnw384 nw384 0 2f
CT1228 t1228 0 0.1f
M3223 t1228 na4 vdd vdd pch w=2u l=180n
M3224 t1228 nw384 vdd vdd pch w=2u l=180n
CT1229 t1229 0 0.1f
M3225 t1228 na4 t1229 0 nch w=1u l=180n
M3226 t1229 nw384 0 0 nch w=1u l=180n
M3227 nw385 t1228 vdd vdd pch w=2u l=180n
M3228 nw385 t1228 0 0 nch w=1u l=180n
Cnw385 nw385 0 2f
CT1230 t1230 0 0.1f
M3229 t1230 nw382 vdd vdd pch w=2u l=180n
M3230 t1230 nw385 vdd vdd pch w=2u l=180n
CT1231 t1231 0 0.1f
M3231 t1230 nw382 t1231 0 nch w=1u l=180n
M3232 t1231 nw385 0 0 nch w=1u l=180n
M3233 nw386 t1230 vdd vdd pch w=2u l=180n
M3234 nw386 t1230 0 0 nch w=1u l=180n
Cnw386 nw386 0 2f
CT1232 t1232 0 0.1f
M3235 t1232 nw381 0 0 nch w=1u l=180n
M3236 t1232 nw386 0 0 nch w=1u l=180n
CT1233 t1233 0 0.1f
M3237 t1233 nw381 vdd vdd pch w=2u l=180n
M3238 t1232 nw386 t1233 vdd pch w=2u l=180n
M3239 nw387 t1232 vdd vdd pch w=2u l=180n
M3240 nw387 t1232 0 0 nch w=1u l=180n
Cnw387 nw387 0 2f
CT1234 t1234 0 0.1f
M3241 t1234 nw382 vdd vdd pch w=2u l=180n
M3242 t1234 nw383 vdd vdd pch w=2u l=180n
CT1235 t1235 0 0.1f
M3243 t1234 nw382 t1235 0 nch w=1u l=180n
M3244 t1235 nw383 0 0 nch w=1u l=180n
M3245 nw388 t1234 vdd vdd pch w=2u l=180n
M3246 nw388 t1234 0 0 nch w=1u l=180n
Cnw388 nw388 0 2f
CT1236 t1236 0 0.1f
CT1237 t1237 0 0.1f
CT1238 t1238 0 0.1f
M3247 t1236 na3 vdd vdd pch w=2u l=180n
M3248 t1236 nb3 vdd vdd pch w=2u l=180n
CT1239 t1239 0 0.1f
M3249 t1236 na3 t1239 0 nch w=1u l=180n
M3250 t1239 nb3 0 0 nch w=1u l=180n
M3251 t1237 na3 vdd vdd pch w=2u l=180n
M3252 t1237 t1236 vdd vdd pch w=2u l=180n
CT1240 t1240 0 0.1f
M3253 t1237 na3 t1240 0 nch w=1u l=180n
M3254 t1240 t1236 0 0 nch w=1u l=180n
M3255 t1238 nb3 vdd vdd pch w=2u l=180n
M3256 t1238 t1236 vdd vdd pch w=2u l=180n
CT1241 t1241 0 0.1f
M3257 t1238 nb3 t1241 0 nch w=1u l=180n
M3258 t1241 t1236 0 0 nch w=1u l=180n
CT1242 t1242 0 0.1f
M3259 t1242 t1237 vdd vdd pch w=2u l=180n
M3260 t1242 t1238 vdd vdd pch w=2u l=180n
CT1243 t1243 0 0.1f
M3261 t1242 t1237 t1243 0 nch w=1u l=180n
M3262 t1243 t1238 0 0 nch w=1u l=180n
M3263 nw389 t1242 vdd vdd pch w=2u l=180n
M3264 nw389 t1242 0 0 nch w=1u l=180n
Cnw389 nw389 0 2f
M3265 nw390 nb3 vdd vdd pch w=2u l=180n
M3266 nw390 nb3 0 0 nch w=1u l=180n
Cnw390 nw390 0 2f
CT1244 t1244 0 0.1f
M3267 t1244 na3 vdd vdd pch w=2u l=180n
M3268 t1244 nw390 vdd vdd pch w=2u l=180n
CT1245 t1245 0 0.1f
M3269 t1244 na3 t1245 0 nch w=1u l=180n
M3270 t1245 nw390 0 0 nch w=1u l=180n
M3271 nw391 t1244 vdd vdd pch w=2u l=180n
M3272 nw391 t1244 0 0 nch w=1u l=180n
Cnw391 nw391 0 2f
CT1246 t1246 0 0.1f
M3273 t1246 nw388 vdd vdd pch w=2u l=180n
M3274 t1246 nw391 vdd vdd pch w=2u l=180n
CT1247 t1247 0 0.1f
M3275 t1246 nw388 t1247 0 nch w=1u l=180n
M3276 t1247 nw391 0 0 nch w=1u l=180n
M3277 nw392 t1246 vdd vdd pch w=2u l=180n
M3278 nw392 t1246 0 0 nch w=1u l=180n
Cnw392 nw392 0 2f
CT1248 t1248 0 0.1f
M3279 t1248 nw387 0 0 nch w=1u l=180n
M3280 t1248 nw392 0 0 nch w=1u l=180n
CT1249 t1249 0 0.1f
M3281 t1249 nw387 vdd vdd pch w=2u l=180n
M3282 t1248 nw392 t1249 vdd pch w=2u l=180n
M3283 nw393 t1248 vdd vdd pch w=2u l=180n
M3284 nw393 t1248 0 0 nch w=1u l=180n
Cnw393 nw393 0 2f
CT1250 t1250 0 0.1f
M3285 t1250 nw388 vdd vdd pch w=2u l=180n
M3286 t1250 nw389 vdd vdd pch w=2u l=180n
CT1251 t1251 0 0.1f
M3287 t1250 nw388 t1251 0 nch w=1u l=180n
M3288 t1251 nw389 0 0 nch w=1u l=180n
M3289 nw394 t1250 vdd vdd pch w=2u l=180n
M3290 nw394 t1250 0 0 nch w=1u l=180n
Cnw394 nw394 0 2f
CT1252 t1252 0 0.1f
CT1253 t1253 0 0.1f
CT1254 t1254 0 0.1f
M3291 t1252 na2 vdd vdd pch w=2u l=180n
M3292 t1252 nb2 vdd vdd pch w=2u l=180n
CT1255 t1255 0 0.1f
M3293 t1252 na2 t1255 0 nch w=1u l=180n
M3294 t1255 nb2 0 0 nch w=1u l=180n
M3295 t1253 na2 vdd vdd pch w=2u l=180n
M3296 t1253 t1252 vdd vdd pch w=2u l=180n
CT1256 t1256 0 0.1f
M3297 t1253 na2 t1256 0 nch w=1u l=180n
M3298 t1256 t1252 0 0 nch w=1u l=180n
M3299 t1254 nb2 vdd vdd pch w=2u l=180n
M3300 t1254 t1252 vdd vdd pch w=2u l=180n
CT1257 t1257 0 0.1f
M3301 t1254 nb2 t1257 0 nch w=1u l=180n
M3302 t1257 t1252 0 0 nch w=1u l=180n
CT1258 t1258 0 0.1f
M3303 t1258 t1253 vdd vdd pch w=2u l=180n
M3304 t1258 t1254 vdd vdd pch w=2u l=180n
CT1259 t1259 0 0.1f
M3305 t1258 t1253 t1259 0 nch w=1u l=180n
M3306 t1259 t1254 0 0 nch w=1u l=180n
M3307 nw395 t1258 vdd vdd pch w=2u l=180n
M3308 nw395 t1258 0 0 nch w=1u l=180n
Cnw395 nw395 0 2f
M3309 nw396 nb2 vdd vdd pch w=2u l=180n
M3310 nw396 nb2 0 0 nch w=1u l=180n
Cnw396 nw396 0 2f
CT1260 t1260 0 0.1f
M3311 t1260 na2 vdd vdd pch w=2u l=180n
M3312 t1260 nw396 vdd vdd pch w=2u l=180n
CT1261 t1261 0 0.1f
M3313 t1260 na2 t1261 0 nch w=1u l=180n
M3314 t1261 nw396 0 0 nch w=1u l=180n
M3315 nw397 t1260 vdd vdd pch w=2u l=180n
M3316 nw397 t1260 0 0 nch w=1u l=180n
Cnw397 nw397 0 2f
CT1262 t1262 0 0.1f
M3317 t1262 nw394 vdd vdd pch w=2u l=180n
M3318 t1262 nw397 vdd vdd pch w=2u l=180n
CT1263 t1263 0 0.1f
M3319 t1262 nw394 t1263 0 nch w=1u l=180n
M3320 t1263 nw397 0 0 nch w=1u l=180n
M3321 nw398 t1262 vdd vdd pch w=2u l=180n
M3322 nw398 t1262 0 0 nch w=1u l=180n
Cnw398 nw398 0 2f
CT1264 t1264 0 0.1f
M3323 t1264 nw393 0 0 nch w=1u l=180n
M3324 t1264 nw398 0 0 nch w=1u l=180n
CT1265 t1265 0 0.1f
M3325 t1265 nw393 vdd vdd pch w=2u l=180n
M3326 t1264 nw398 t1265 vdd pch w=2u l=180n
M3327 nw399 t1264 vdd vdd pch w=2u l=180n
M3328 nw399 t1264 0 0 nch w=1u l=180n
Cnw399 nw399 0 2f
CT1266 t1266 0 0.1f
M3329 t1266 nw394 vdd vdd pch w=2u l=180n
M3330 t1266 nw395 vdd vdd pch w=2u l=180n
CT1267 t1267 0 0.1f
M3331 t1266 nw394 t1267 0 nch w=1u l=180n
M3332 t1267 nw395 0 0 nch w=1u l=180n
M3333 nw400 t1266 vdd vdd pch w=2u l=180n
M3334 nw400 t1266 0 0 nch w=1u l=180n
Cnw400 nw400 0 2f
CT1268 t1268 0 0.1f
CT1269 t1269 0 0.1f
CT1270 t1270 0 0.1f
M3335 t1268 na1 vdd vdd pch w=2u l=180n
M3336 t1268 nb1 vdd vdd pch w=2u l=180n
CT1271 t1271 0 0.1f
M3337 t1268 na1 t1271 0 nch w=1u l=180n
M3338 t1271 nb1 0 0 nch w=1u l=180n
M3339 t1269 na1 vdd vdd pch w=2u l=180n
M3340 t1269 t1268 vdd vdd pch w=2u l=180n
CT1272 t1272 0 0.1f
M3341 t1269 na1 t1272 0 nch w=1u l=180n
M3342 t1272 t1268 0 0 nch w=1u l=180n
M3343 t1270 nb1 vdd vdd pch w=2u l=180n
M3344 t1270 t1268 vdd vdd pch w=2u l=180n
CT1273 t1273 0 0.1f
M3345 t1270 nb1 t1273 0 nch w=1u l=180n
M3346 t1273 t1268 0 0 nch w=1u l=180n
CT1274 t1274 0 0.1f
M3347 t1274 t1269 vdd vdd pch w=2u l=180n
M3348 t1274 t1270 vdd vdd pch w=2u l=180n
CT1275 t1275 0 0.1f
M3349 t1274 t1269 t1275 0 nch w=1u l=180n
M3350 t1275 t1270 0 0 nch w=1u l=180n
M3351 nw401 t1274 vdd vdd pch w=2u l=180n
M3352 nw401 t1274 0 0 nch w=1u l=180n
Cnw401 nw401 0 2f
M3353 nw402 nb1 vdd vdd pch w=2u l=180n
M3354 nw402 nb1 0 0 nch w=1u l=180n
Cnw402 nw402 0 2f
CT1276 t1276 0 0.1f
M3355 t1276 na1 vdd vdd pch w=2u l=180n
M3356 t1276 nw402 vdd vdd pch w=2u l=180n
CT1277 t1277 0 0.1f
M3357 t1276 na1 t1277 0 nch w=1u l=180n
M3358 t1277 nw402 0 0 nch w=1u l=180n
M3359 nw403 t1276 vdd vdd pch w=2u l=180n
M3360 nw403 t1276 0 0 nch w=1u l=180n
Cnw403 nw403 0 2f
CT1278 t1278 0 0.1f
M3361 t1278 nw400 vdd vdd pch w=2u l=180n
M3362 t1278 nw403 vdd vdd pch w=2u l=180n
CT1279 t1279 0 0.1f
M3363 t1278 nw400 t1279 0 nch w=1u l=180n
M3364 t1279 nw403 0 0 nch w=1u l=180n
M3365 nw404 t1278 vdd vdd pch w=2u l=180n
M3366 nw404 t1278 0 0 nch w=1u l=180n
Cnw404 nw404 0 2f
CT1280 t1280 0 0.1f
M3367 t1280 nw399 0 0 nch w=1u l=180n
M3368 t1280 nw404 0 0 nch w=1u l=180n
CT1281 t1281 0 0.1f
M3369 t1281 nw399 vdd vdd pch w=2u l=180n
M3370 t1280 nw404 t1281 vdd pch w=2u l=180n
M3371 nw405 t1280 vdd vdd pch w=2u l=180n
M3372 nw405 t1280 0 0 nch w=1u l=180n
Cnw405 nw405 0 2f
CT1282 t1282 0 0.1f
M3373 t1282 nw400 vdd vdd pch w=2u l=180n
M3374 t1282 nw401 vdd vdd pch w=2u l=180n
CT1283 t1283 0 0.1f
M3375 t1282 nw400 t1283 0 nch w=1u l=180n
M3376 t1283 nw401 0 0 nch w=1u l=180n
M3377 nw406 t1282 vdd vdd pch w=2u l=180n
M3378 nw406 t1282 0 0 nch w=1u l=180n
Cnw406 nw406 0 2f
CT1284 t1284 0 0.1f
CT1285 t1285 0 0.1f
CT1286 t1286 0 0.1f
M3379 t1284 na0 vdd vdd pch w=2u l=180n
M3380 t1284 nb0 vdd vdd pch w=2u l=180n
CT1287 t1287 0 0.1f
M3381 t1284 na0 t1287 0 nch w=1u l=180n
M3382 t1287 nb0 0 0 nch w=1u l=180n
M3383 t1285 na0 vdd vdd pch w=2u l=180n
M3384 t1285 t1284 vdd vdd pch w=2u l=180n
CT1288 t1288 0 0.1f
M3385 t1285 na0 t1288 0 nch w=1u l=180n
M3386 t1288 t1284 0 0 nch w=1u l=180n
M3387 t1286 nb0 vdd vdd pch w=2u l=180n
M3388 t1286 t1284 vdd vdd pch w=2u l=180n
CT1289 t1289 0 0.1f
M3389 t1286 nb0 t1289 0 nch w=1u l=180n
M3390 t1289 t1284 0 0 nch w=1u l=180n
CT1290 t1290 0 0.1f
M3391 t1290 t1285 vdd vdd pch w=2u l=180n
M3392 t1290 t1286 vdd vdd pch w=2u l=180n
CT1291 t1291 0 0.1f
M3393 t1290 t1285 t1291 0 nch w=1u l=180n
M3394 t1291 t1286 0 0 nch w=1u l=180n
M3395 nw407 t1290 vdd vdd pch w=2u l=180n
M3396 nw407 t1290 0 0 nch w=1u l=180n
Cnw407 nw407 0 2f
M3397 nw408 nb0 vdd vdd pch w=2u l=180n
M3398 nw408 nb0 0 0 nch w=1u l=180n
Cnw408 nw408 0 2f
CT1292 t1292 0 0.1f
M3399 t1292 na0 vdd vdd pch w=2u l=180n
M3400 t1292 nw408 vdd vdd pch w=2u l=180n
CT1293 t1293 0 0.1f
M3401 t1292 na0 t1293 0 nch w=1u l=180n
M3402 t1293 nw408 0 0 nch w=1u l=180n
M3403 nw409 t1292 vdd vdd pch w=2u l=180n
M3404 nw409 t1292 0 0 nch w=1u l=180n
Cnw409 nw409 0 2f
CT1294 t1294 0 0.1f
M3405 t1294 nw406 vdd vdd pch w=2u l=180n
M3406 t1294 nw409 vdd vdd pch w=2u l=180n
CT1295 t1295 0 0.1f
M3407 t1294 nw406 t1295 0 nch w=1u l=180n
M3408 t1295 nw409 0 0 nch w=1u l=180n
M3409 nw410 t1294 vdd vdd pch w=2u l=180n
M3410 nw410 t1294 0 0 nch w=1u l=180n
Cnw410 nw410 0 2f
CT1296 t1296 0 0.1f
M3411 t1296 nw405 0 0 nch w=1u l=180n
M3412 t1296 nw410 0 0 nch w=1u l=180n
CT1297 t1297 0 0.1f
M3413 t1297 nw405 vdd vdd pch w=2u l=180n
M3414 t1296 nw410 t1297 vdd pch w=2u l=180n
M3415 nw411 t1296 vdd vdd pch w=2u l=180n
M3416 nw411 t1296 0 0 nch w=1u l=180n
Cnw411 nw411 0 2f
CT1298 t1298 0 0.1f
M3417 t1298 nw406 vdd vdd pch w=2u l=180n
M3418 t1298 nw407 vdd vdd pch w=2u l=180n
CT1299 t1299 0 0.1f
M3419 t1298 nw406 t1299 0 nch w=1u l=180n
M3420 t1299 nw407 0 0 nch w=1u l=180n
M3421 nw412 t1298 vdd vdd pch w=2u l=180n
M3422 nw412 t1298 0 0 nch w=1u l=180n
Cnw412 nw412 0 2f
CT1300 t1300 0 0.1f
M3423 t1300 nw221 vdd vdd pch w=2u l=180n
M3424 t1300 nw221 0 0 nch w=1u l=180n
M3425 ncout t1300 vdd vdd pch w=2u l=180n
M3426 ncout t1300 0 0 nch w=1u l=180n
Cncout ncout 0 2f
CT1301 t1301 0 0.1f
M3427 t1301 nw223 vdd vdd pch w=2u l=180n
M3428 t1301 nw223 0 0 nch w=1u l=180n
M3429 nparity t1301 vdd vdd pch w=2u l=180n
M3430 nparity t1301 0 0 nch w=1u l=180n
Cnparity nparity 0 2f
CT1302 t1302 0 0.1f
M3431 t1302 nw411 vdd vdd pch w=2u l=180n
M3432 t1302 nw411 0 0 nch w=1u l=180n
M3433 na_gt_b t1302 vdd vdd pch w=2u l=180n
M3434 na_gt_b t1302 0 0 nch w=1u l=180n
Cna_gt_b na_gt_b 0 2f
CT1303 t1303 0 0.1f
M3435 t1303 nw412 vdd vdd pch w=2u l=180n
M3436 t1303 nw412 0 0 nch w=1u l=180n
M3437 na_eq_b t1303 vdd vdd pch w=2u l=180n
M3438 na_eq_b t1303 0 0 nch w=1u l=180n
Cna_eq_b na_eq_b 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: ns0 ns1 ns2 ns3 ns4 ns5 ns6 ns7 ns8 ns9 ns10 ns11 ns12 ns13 ns14 ns15 ns16 ns17 ns18 ns19 ns20 ns21 ns22 ns23 ns24 ns25 ns26 ns27 ns28 ns29 ns30 ns31 ncout nparity na_gt_b na_eq_b
.end
