* s1423 (s1423: 74 flip-flops, 657 gates): 756 gates, 5980 transistors
VDD vdd 0 DC 1.8
VIN0 ni0 0 PULSE(0 1.8 5e-10 20p 20p 1e-09 2e-09)
VIN1 ni1 0 PULSE(0 1.8 1e-09 20p 20p 2e-09 4e-09)
VIN2 ni2 0 PULSE(0 1.8 2e-09 20p 20p 4e-09 8e-09)
VIN3 ni3 0 PULSE(0 1.8 4e-09 20p 20p 8e-09 1.6e-08)
VIN4 ni4 0 PULSE(0 1.8 8e-09 20p 20p 1.6e-08 3.2e-08)
VIN5 ni5 0 PULSE(0 1.8 1.6e-08 20p 20p 3.2e-08 6.4e-08)
VIN6 ni6 0 PULSE(0 1.8 3.2e-08 20p 20p 6.4e-08 1.28e-07)
VIN7 ni7 0 PULSE(0 1.8 6.4e-08 20p 20p 1.28e-07 2.56e-07)
VIN8 ni8 0 PULSE(0 1.8 1.28e-07 20p 20p 2.56e-07 5.12e-07)
VIN9 ni9 0 PULSE(0 1.8 2.56e-07 20p 20p 5.12e-07 1.024e-06)
VIN10 ni10 0 PULSE(0 1.8 5.12e-07 20p 20p 1.024e-06 2.048e-06)
VIN11 ni11 0 PULSE(0 1.8 1.024e-06 20p 20p 2.048e-06 4.096e-06)
VIN12 ni12 0 PULSE(0 1.8 2.048e-06 20p 20p 4.096e-06 8.192e-06)
VIN13 ni13 0 PULSE(0 1.8 4.096e-06 20p 20p 8.192e-06 1.6384e-05)
VIN14 ni14 0 PULSE(0 1.8 8.192e-06 20p 20p 1.6384e-05 3.2768e-05)
VIN15 ni15 0 PULSE(0 1.8 1.6384e-05 20p 20p 3.2768e-05 6.5536e-05)
VIN16 nq0 0 PULSE(0 1.8 3.2768e-05 20p 20p 6.5536e-05 0.000131072)
VIN17 nq1 0 PULSE(0 1.8 6.5536e-05 20p 20p 0.000131072 0.000262144)
VIN18 nq2 0 PULSE(0 1.8 0.000131072 20p 20p 0.000262144 0.000524288)
VIN19 nq3 0 PULSE(0 1.8 0.000262144 20p 20p 0.000524288 0.001048576)
VIN20 nq4 0 PULSE(0 1.8 0.000524288 20p 20p 0.001048576 0.002097152)
VIN21 nq5 0 PULSE(0 1.8 0.001048576 20p 20p 0.002097152 0.004194304)
VIN22 nq6 0 PULSE(0 1.8 0.002097152 20p 20p 0.004194304 0.008388608)
VIN23 nq7 0 PULSE(0 1.8 0.004194304 20p 20p 0.008388608 0.016777216)
VIN24 nq8 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN25 nq9 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN26 nq10 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN27 nq11 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN28 nq12 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN29 nq13 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN30 nq14 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN31 nq15 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN32 nq16 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN33 nq17 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN34 nq18 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN35 nq19 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN36 nq20 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN37 nq21 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN38 nq22 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN39 nq23 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN40 nq24 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN41 nq25 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN42 nq26 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN43 nq27 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN44 nq28 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN45 nq29 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN46 nq30 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN47 nq31 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN48 nq32 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN49 nq33 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN50 nq34 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN51 nq35 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN52 nq36 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN53 nq37 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN54 nq38 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN55 nq39 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN56 nq40 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN57 nq41 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN58 nq42 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN59 nq43 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN60 nq44 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN61 nq45 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN62 nq46 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN63 nq47 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN64 nq48 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN65 nq49 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN66 nq50 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN67 nq51 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN68 nq52 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN69 nq53 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN70 nq54 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN71 nq55 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN72 nq56 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN73 nq57 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN74 nq58 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN75 nq59 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN76 nq60 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN77 nq61 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN78 nq62 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN79 nq63 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN80 nq64 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN81 nq65 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN82 nq66 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN83 nq67 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN84 nq68 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN85 nq69 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN86 nq70 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN87 nq71 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN88 nq72 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN89 nq73 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
CT1 t1 0 0.1f
CT2 t2 0 0.1f
CT3 t3 0 0.1f
M1 t1 nq0 vdd vdd pch w=2u l=180n
M2 t1 ni0 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M3 t1 nq0 t4 0 nch w=1u l=180n
M4 t4 ni0 0 0 nch w=1u l=180n
M5 t2 nq0 vdd vdd pch w=2u l=180n
M6 t2 t1 vdd vdd pch w=2u l=180n
CT5 t5 0 0.1f
M7 t2 nq0 t5 0 nch w=1u l=180n
M8 t5 t1 0 0 nch w=1u l=180n
M9 t3 ni0 vdd vdd pch w=2u l=180n
M10 t3 t1 vdd vdd pch w=2u l=180n
CT6 t6 0 0.1f
M11 t3 ni0 t6 0 nch w=1u l=180n
M12 t6 t1 0 0 nch w=1u l=180n
M13 nw1 t2 vdd vdd pch w=2u l=180n
M14 nw1 t3 vdd vdd pch w=2u l=180n
CT7 t7 0 0.1f
M15 nw1 t2 t7 0 nch w=1u l=180n
M16 t7 t3 0 0 nch w=1u l=180n
Cnw1 nw1 0 2f
CT8 t8 0 0.1f
M17 t8 ni0 vdd vdd pch w=2u l=180n
M18 t8 nq0 vdd vdd pch w=2u l=180n
CT9 t9 0 0.1f
M19 t8 ni0 t9 0 nch w=1u l=180n
M20 t9 nq0 0 0 nch w=1u l=180n
M21 nw2 t8 vdd vdd pch w=2u l=180n
M22 nw2 t8 0 0 nch w=1u l=180n
Cnw2 nw2 0 2f
CT10 t10 0 0.1f
CT11 t11 0 0.1f
CT12 t12 0 0.1f
M23 t10 nq1 vdd vdd pch w=2u l=180n
M24 t10 nw2 vdd vdd pch w=2u l=180n
CT13 t13 0 0.1f
M25 t10 nq1 t13 0 nch w=1u l=180n
M26 t13 nw2 0 0 nch w=1u l=180n
M27 t11 nq1 vdd vdd pch w=2u l=180n
M28 t11 t10 vdd vdd pch w=2u l=180n
CT14 t14 0 0.1f
M29 t11 nq1 t14 0 nch w=1u l=180n
M30 t14 t10 0 0 nch w=1u l=180n
M31 t12 nw2 vdd vdd pch w=2u l=180n
M32 t12 t10 vdd vdd pch w=2u l=180n
CT15 t15 0 0.1f
M33 t12 nw2 t15 0 nch w=1u l=180n
M34 t15 t10 0 0 nch w=1u l=180n
M35 nw3 t11 vdd vdd pch w=2u l=180n
M36 nw3 t12 vdd vdd pch w=2u l=180n
CT16 t16 0 0.1f
M37 nw3 t11 t16 0 nch w=1u l=180n
M38 t16 t12 0 0 nch w=1u l=180n
Cnw3 nw3 0 2f
CT17 t17 0 0.1f
M39 t17 nw2 vdd vdd pch w=2u l=180n
M40 t17 nq1 vdd vdd pch w=2u l=180n
CT18 t18 0 0.1f
M41 t17 nw2 t18 0 nch w=1u l=180n
M42 t18 nq1 0 0 nch w=1u l=180n
M43 nw4 t17 vdd vdd pch w=2u l=180n
M44 nw4 t17 0 0 nch w=1u l=180n
Cnw4 nw4 0 2f
CT19 t19 0 0.1f
CT20 t20 0 0.1f
CT21 t21 0 0.1f
M45 t19 nq2 vdd vdd pch w=2u l=180n
M46 t19 nw4 vdd vdd pch w=2u l=180n
CT22 t22 0 0.1f
M47 t19 nq2 t22 0 nch w=1u l=180n
M48 t22 nw4 0 0 nch w=1u l=180n
M49 t20 nq2 vdd vdd pch w=2u l=180n
M50 t20 t19 vdd vdd pch w=2u l=180n
CT23 t23 0 0.1f
M51 t20 nq2 t23 0 nch w=1u l=180n
M52 t23 t19 0 0 nch w=1u l=180n
M53 t21 nw4 vdd vdd pch w=2u l=180n
M54 t21 t19 vdd vdd pch w=2u l=180n
CT24 t24 0 0.1f
M55 t21 nw4 t24 0 nch w=1u l=180n
M56 t24 t19 0 0 nch w=1u l=180n
M57 nw5 t20 vdd vdd pch w=2u l=180n
M58 nw5 t21 vdd vdd pch w=2u l=180n
CT25 t25 0 0.1f
M59 nw5 t20 t25 0 nch w=1u l=180n
M60 t25 t21 0 0 nch w=1u l=180n
Cnw5 nw5 0 2f
CT26 t26 0 0.1f
M61 t26 nw4 vdd vdd pch w=2u l=180n
M62 t26 nq2 vdd vdd pch w=2u l=180n
CT27 t27 0 0.1f
M63 t26 nw4 t27 0 nch w=1u l=180n
M64 t27 nq2 0 0 nch w=1u l=180n
M65 nw6 t26 vdd vdd pch w=2u l=180n
M66 nw6 t26 0 0 nch w=1u l=180n
Cnw6 nw6 0 2f
CT28 t28 0 0.1f
CT29 t29 0 0.1f
CT30 t30 0 0.1f
M67 t28 nq3 vdd vdd pch w=2u l=180n
M68 t28 nw6 vdd vdd pch w=2u l=180n
CT31 t31 0 0.1f
M69 t28 nq3 t31 0 nch w=1u l=180n
M70 t31 nw6 0 0 nch w=1u l=180n
M71 t29 nq3 vdd vdd pch w=2u l=180n
M72 t29 t28 vdd vdd pch w=2u l=180n
CT32 t32 0 0.1f
M73 t29 nq3 t32 0 nch w=1u l=180n
M74 t32 t28 0 0 nch w=1u l=180n
M75 t30 nw6 vdd vdd pch w=2u l=180n
M76 t30 t28 vdd vdd pch w=2u l=180n
CT33 t33 0 0.1f
M77 t30 nw6 t33 0 nch w=1u l=180n
M78 t33 t28 0 0 nch w=1u l=180n
M79 nw7 t29 vdd vdd pch w=2u l=180n
M80 nw7 t30 vdd vdd pch w=2u l=180n
CT34 t34 0 0.1f
M81 nw7 t29 t34 0 nch w=1u l=180n
M82 t34 t30 0 0 nch w=1u l=180n
Cnw7 nw7 0 2f
CT35 t35 0 0.1f
M83 t35 nw6 vdd vdd pch w=2u l=180n
M84 t35 nq3 vdd vdd pch w=2u l=180n
CT36 t36 0 0.1f
M85 t35 nw6 t36 0 nch w=1u l=180n
M86 t36 nq3 0 0 nch w=1u l=180n
M87 nw8 t35 vdd vdd pch w=2u l=180n
M88 nw8 t35 0 0 nch w=1u l=180n
Cnw8 nw8 0 2f
CT37 t37 0 0.1f
CT38 t38 0 0.1f
CT39 t39 0 0.1f
M89 t37 nq4 vdd vdd pch w=2u l=180n
M90 t37 nw8 vdd vdd pch w=2u l=180n
CT40 t40 0 0.1f
M91 t37 nq4 t40 0 nch w=1u l=180n
M92 t40 nw8 0 0 nch w=1u l=180n
M93 t38 nq4 vdd vdd pch w=2u l=180n
M94 t38 t37 vdd vdd pch w=2u l=180n
CT41 t41 0 0.1f
M95 t38 nq4 t41 0 nch w=1u l=180n
M96 t41 t37 0 0 nch w=1u l=180n
M97 t39 nw8 vdd vdd pch w=2u l=180n
M98 t39 t37 vdd vdd pch w=2u l=180n
CT42 t42 0 0.1f
M99 t39 nw8 t42 0 nch w=1u l=180n
M100 t42 t37 0 0 nch w=1u l=180n
M101 nw9 t38 vdd vdd pch w=2u l=180n
M102 nw9 t39 vdd vdd pch w=2u l=180n
CT43 t43 0 0.1f
M103 nw9 t38 t43 0 nch w=1u l=180n
M104 t43 t39 0 0 nch w=1u l=180n
Cnw9 nw9 0 2f
CT44 t44 0 0.1f
M105 t44 nw8 vdd vdd pch w=2u l=180n
M106 t44 nq4 vdd vdd pch w=2u l=180n
CT45 t45 0 0.1f
M107 t44 nw8 t45 0 nch w=1u l=180n
M108 t45 nq4 0 0 nch w=1u l=180n
M109 nw10 t44 vdd vdd pch w=2u l=180n
M110 nw10 t44 0 0 nch w=1u l=180n
Cnw10 nw10 0 2f
CT46 t46 0 0.1f
CT47 t47 0 0.1f
CT48 t48 0 0.1f
M111 t46 nq5 vdd vdd pch w=2u l=180n
M112 t46 nw10 vdd vdd pch w=2u l=180n
CT49 t49 0 0.1f
M113 t46 nq5 t49 0 nch w=1u l=180n
M114 t49 nw10 0 0 nch w=1u l=180n
M115 t47 nq5 vdd vdd pch w=2u l=180n
M116 t47 t46 vdd vdd pch w=2u l=180n
CT50 t50 0 0.1f
M117 t47 nq5 t50 0 nch w=1u l=180n
M118 t50 t46 0 0 nch w=1u l=180n
M119 t48 nw10 vdd vdd pch w=2u l=180n
M120 t48 t46 vdd vdd pch w=2u l=180n
CT51 t51 0 0.1f
M121 t48 nw10 t51 0 nch w=1u l=180n
M122 t51 t46 0 0 nch w=1u l=180n
M123 nw11 t47 vdd vdd pch w=2u l=180n
M124 nw11 t48 vdd vdd pch w=2u l=180n
CT52 t52 0 0.1f
M125 nw11 t47 t52 0 nch w=1u l=180n
M126 t52 t48 0 0 nch w=1u l=180n
Cnw11 nw11 0 2f
CT53 t53 0 0.1f
M127 t53 nw10 vdd vdd pch w=2u l=180n
M128 t53 nq5 vdd vdd pch w=2u l=180n
CT54 t54 0 0.1f
M129 t53 nw10 t54 0 nch w=1u l=180n
M130 t54 nq5 0 0 nch w=1u l=180n
M131 nw12 t53 vdd vdd pch w=2u l=180n
M132 nw12 t53 0 0 nch w=1u l=180n
Cnw12 nw12 0 2f
CT55 t55 0 0.1f
CT56 t56 0 0.1f
CT57 t57 0 0.1f
M133 t55 nq6 vdd vdd pch w=2u l=180n
M134 t55 nw12 vdd vdd pch w=2u l=180n
CT58 t58 0 0.1f
M135 t55 nq6 t58 0 nch w=1u l=180n
M136 t58 nw12 0 0 nch w=1u l=180n
M137 t56 nq6 vdd vdd pch w=2u l=180n
M138 t56 t55 vdd vdd pch w=2u l=180n
CT59 t59 0 0.1f
M139 t56 nq6 t59 0 nch w=1u l=180n
M140 t59 t55 0 0 nch w=1u l=180n
M141 t57 nw12 vdd vdd pch w=2u l=180n
M142 t57 t55 vdd vdd pch w=2u l=180n
CT60 t60 0 0.1f
M143 t57 nw12 t60 0 nch w=1u l=180n
M144 t60 t55 0 0 nch w=1u l=180n
M145 nw13 t56 vdd vdd pch w=2u l=180n
M146 nw13 t57 vdd vdd pch w=2u l=180n
CT61 t61 0 0.1f
M147 nw13 t56 t61 0 nch w=1u l=180n
M148 t61 t57 0 0 nch w=1u l=180n
Cnw13 nw13 0 2f
CT62 t62 0 0.1f
M149 t62 nw12 vdd vdd pch w=2u l=180n
M150 t62 nq6 vdd vdd pch w=2u l=180n
CT63 t63 0 0.1f
M151 t62 nw12 t63 0 nch w=1u l=180n
M152 t63 nq6 0 0 nch w=1u l=180n
M153 nw14 t62 vdd vdd pch w=2u l=180n
M154 nw14 t62 0 0 nch w=1u l=180n
Cnw14 nw14 0 2f
CT64 t64 0 0.1f
CT65 t65 0 0.1f
CT66 t66 0 0.1f
M155 t64 nq7 vdd vdd pch w=2u l=180n
M156 t64 nw14 vdd vdd pch w=2u l=180n
CT67 t67 0 0.1f
M157 t64 nq7 t67 0 nch w=1u l=180n
M158 t67 nw14 0 0 nch w=1u l=180n
M159 t65 nq7 vdd vdd pch w=2u l=180n
M160 t65 t64 vdd vdd pch w=2u l=180n
CT68 t68 0 0.1f
M161 t65 nq7 t68 0 nch w=1u l=180n
M162 t68 t64 0 0 nch w=1u l=180n
M163 t66 nw14 vdd vdd pch w=2u l=180n
M164 t66 t64 vdd vdd pch w=2u l=180n
CT69 t69 0 0.1f
M165 t66 nw14 t69 0 nch w=1u l=180n
M166 t69 t64 0 0 nch w=1u l=180n
M167 nw15 t65 vdd vdd pch w=2u l=180n
M168 nw15 t66 vdd vdd pch w=2u l=180n
CT70 t70 0 0.1f
M169 nw15 t65 t70 0 nch w=1u l=180n
M170 t70 t66 0 0 nch w=1u l=180n
Cnw15 nw15 0 2f
CT71 t71 0 0.1f
M171 t71 nw14 vdd vdd pch w=2u l=180n
M172 t71 nq7 vdd vdd pch w=2u l=180n
CT72 t72 0 0.1f
M173 t71 nw14 t72 0 nch w=1u l=180n
M174 t72 nq7 0 0 nch w=1u l=180n
M175 nw16 t71 vdd vdd pch w=2u l=180n
M176 nw16 t71 0 0 nch w=1u l=180n
Cnw16 nw16 0 2f
CT73 t73 0 0.1f
CT74 t74 0 0.1f
CT75 t75 0 0.1f
M177 t73 nq8 vdd vdd pch w=2u l=180n
M178 t73 nw16 vdd vdd pch w=2u l=180n
CT76 t76 0 0.1f
M179 t73 nq8 t76 0 nch w=1u l=180n
M180 t76 nw16 0 0 nch w=1u l=180n
M181 t74 nq8 vdd vdd pch w=2u l=180n
M182 t74 t73 vdd vdd pch w=2u l=180n
CT77 t77 0 0.1f
M183 t74 nq8 t77 0 nch w=1u l=180n
M184 t77 t73 0 0 nch w=1u l=180n
M185 t75 nw16 vdd vdd pch w=2u l=180n
M186 t75 t73 vdd vdd pch w=2u l=180n
CT78 t78 0 0.1f
M187 t75 nw16 t78 0 nch w=1u l=180n
M188 t78 t73 0 0 nch w=1u l=180n
M189 nw17 t74 vdd vdd pch w=2u l=180n
M190 nw17 t75 vdd vdd pch w=2u l=180n
CT79 t79 0 0.1f
M191 nw17 t74 t79 0 nch w=1u l=180n
M192 t79 t75 0 0 nch w=1u l=180n
Cnw17 nw17 0 2f
CT80 t80 0 0.1f
M193 t80 nw16 vdd vdd pch w=2u l=180n
M194 t80 nq8 vdd vdd pch w=2u l=180n
CT81 t81 0 0.1f
M195 t80 nw16 t81 0 nch w=1u l=180n
M196 t81 nq8 0 0 nch w=1u l=180n
M197 nw18 t80 vdd vdd pch w=2u l=180n
M198 nw18 t80 0 0 nch w=1u l=180n
Cnw18 nw18 0 2f
CT82 t82 0 0.1f
CT83 t83 0 0.1f
CT84 t84 0 0.1f
M199 t82 nq9 vdd vdd pch w=2u l=180n
M200 t82 nw18 vdd vdd pch w=2u l=180n
CT85 t85 0 0.1f
M201 t82 nq9 t85 0 nch w=1u l=180n
M202 t85 nw18 0 0 nch w=1u l=180n
M203 t83 nq9 vdd vdd pch w=2u l=180n
M204 t83 t82 vdd vdd pch w=2u l=180n
CT86 t86 0 0.1f
M205 t83 nq9 t86 0 nch w=1u l=180n
M206 t86 t82 0 0 nch w=1u l=180n
M207 t84 nw18 vdd vdd pch w=2u l=180n
M208 t84 t82 vdd vdd pch w=2u l=180n
CT87 t87 0 0.1f
M209 t84 nw18 t87 0 nch w=1u l=180n
M210 t87 t82 0 0 nch w=1u l=180n
M211 nw19 t83 vdd vdd pch w=2u l=180n
M212 nw19 t84 vdd vdd pch w=2u l=180n
CT88 t88 0 0.1f
M213 nw19 t83 t88 0 nch w=1u l=180n
M214 t88 t84 0 0 nch w=1u l=180n
Cnw19 nw19 0 2f
CT89 t89 0 0.1f
M215 t89 nw18 vdd vdd pch w=2u l=180n
M216 t89 nq9 vdd vdd pch w=2u l=180n
CT90 t90 0 0.1f
M217 t89 nw18 t90 0 nch w=1u l=180n
M218 t90 nq9 0 0 nch w=1u l=180n
M219 nw20 t89 vdd vdd pch w=2u l=180n
M220 nw20 t89 0 0 nch w=1u l=180n
Cnw20 nw20 0 2f
CT91 t91 0 0.1f
CT92 t92 0 0.1f
CT93 t93 0 0.1f
M221 t91 nq10 vdd vdd pch w=2u l=180n
M222 t91 nw20 vdd vdd pch w=2u l=180n
CT94 t94 0 0.1f
M223 t91 nq10 t94 0 nch w=1u l=180n
M224 t94 nw20 0 0 nch w=1u l=180n
M225 t92 nq10 vdd vdd pch w=2u l=180n
M226 t92 t91 vdd vdd pch w=2u l=180n
CT95 t95 0 0.1f
M227 t92 nq10 t95 0 nch w=1u l=180n
M228 t95 t91 0 0 nch w=1u l=180n
M229 t93 nw20 vdd vdd pch w=2u l=180n
M230 t93 t91 vdd vdd pch w=2u l=180n
CT96 t96 0 0.1f
M231 t93 nw20 t96 0 nch w=1u l=180n
M232 t96 t91 0 0 nch w=1u l=180n
M233 nw21 t92 vdd vdd pch w=2u l=180n
M234 nw21 t93 vdd vdd pch w=2u l=180n
CT97 t97 0 0.1f
M235 nw21 t92 t97 0 nch w=1u l=180n
M236 t97 t93 0 0 nch w=1u l=180n
Cnw21 nw21 0 2f
CT98 t98 0 0.1f
M237 t98 nw20 vdd vdd pch w=2u l=180n
M238 t98 nq10 vdd vdd pch w=2u l=180n
CT99 t99 0 0.1f
M239 t98 nw20 t99 0 nch w=1u l=180n
M240 t99 nq10 0 0 nch w=1u l=180n
M241 nw22 t98 vdd vdd pch w=2u l=180n
M242 nw22 t98 0 0 nch w=1u l=180n
Cnw22 nw22 0 2f
CT100 t100 0 0.1f
CT101 t101 0 0.1f
CT102 t102 0 0.1f
M243 t100 nq11 vdd vdd pch w=2u l=180n
M244 t100 nw22 vdd vdd pch w=2u l=180n
CT103 t103 0 0.1f
M245 t100 nq11 t103 0 nch w=1u l=180n
M246 t103 nw22 0 0 nch w=1u l=180n
M247 t101 nq11 vdd vdd pch w=2u l=180n
M248 t101 t100 vdd vdd pch w=2u l=180n
CT104 t104 0 0.1f
M249 t101 nq11 t104 0 nch w=1u l=180n
M250 t104 t100 0 0 nch w=1u l=180n
M251 t102 nw22 vdd vdd pch w=2u l=180n
M252 t102 t100 vdd vdd pch w=2u l=180n
CT105 t105 0 0.1f
M253 t102 nw22 t105 0 nch w=1u l=180n
M254 t105 t100 0 0 nch w=1u l=180n
M255 nw23 t101 vdd vdd pch w=2u l=180n
M256 nw23 t102 vdd vdd pch w=2u l=180n
CT106 t106 0 0.1f
M257 nw23 t101 t106 0 nch w=1u l=180n
M258 t106 t102 0 0 nch w=1u l=180n
Cnw23 nw23 0 2f
CT107 t107 0 0.1f
M259 t107 nw22 vdd vdd pch w=2u l=180n
M260 t107 nq11 vdd vdd pch w=2u l=180n
CT108 t108 0 0.1f
M261 t107 nw22 t108 0 nch w=1u l=180n
M262 t108 nq11 0 0 nch w=1u l=180n
M263 nw24 t107 vdd vdd pch w=2u l=180n
M264 nw24 t107 0 0 nch w=1u l=180n
Cnw24 nw24 0 2f
CT109 t109 0 0.1f
CT110 t110 0 0.1f
CT111 t111 0 0.1f
M265 t109 nq12 vdd vdd pch w=2u l=180n
M266 t109 nw24 vdd vdd pch w=2u l=180n
CT112 t112 0 0.1f
M267 t109 nq12 t112 0 nch w=1u l=180n
M268 t112 nw24 0 0 nch w=1u l=180n
M269 t110 nq12 vdd vdd pch w=2u l=180n
M270 t110 t109 vdd vdd pch w=2u l=180n
CT113 t113 0 0.1f
M271 t110 nq12 t113 0 nch w=1u l=180n
M272 t113 t109 0 0 nch w=1u l=180n
M273 t111 nw24 vdd vdd pch w=2u l=180n
M274 t111 t109 vdd vdd pch w=2u l=180n
CT114 t114 0 0.1f
M275 t111 nw24 t114 0 nch w=1u l=180n
M276 t114 t109 0 0 nch w=1u l=180n
M277 nw25 t110 vdd vdd pch w=2u l=180n
M278 nw25 t111 vdd vdd pch w=2u l=180n
CT115 t115 0 0.1f
M279 nw25 t110 t115 0 nch w=1u l=180n
M280 t115 t111 0 0 nch w=1u l=180n
Cnw25 nw25 0 2f
CT116 t116 0 0.1f
M281 t116 nw24 vdd vdd pch w=2u l=180n
M282 t116 nq12 vdd vdd pch w=2u l=180n
CT117 t117 0 0.1f
M283 t116 nw24 t117 0 nch w=1u l=180n
M284 t117 nq12 0 0 nch w=1u l=180n
M285 nw26 t116 vdd vdd pch w=2u l=180n
M286 nw26 t116 0 0 nch w=1u l=180n
Cnw26 nw26 0 2f
CT118 t118 0 0.1f
CT119 t119 0 0.1f
CT120 t120 0 0.1f
M287 t118 nq13 vdd vdd pch w=2u l=180n
M288 t118 nw26 vdd vdd pch w=2u l=180n
CT121 t121 0 0.1f
M289 t118 nq13 t121 0 nch w=1u l=180n
M290 t121 nw26 0 0 nch w=1u l=180n
M291 t119 nq13 vdd vdd pch w=2u l=180n
M292 t119 t118 vdd vdd pch w=2u l=180n
CT122 t122 0 0.1f
M293 t119 nq13 t122 0 nch w=1u l=180n
M294 t122 t118 0 0 nch w=1u l=180n
M295 t120 nw26 vdd vdd pch w=2u l=180n
M296 t120 t118 vdd vdd pch w=2u l=180n
CT123 t123 0 0.1f
M297 t120 nw26 t123 0 nch w=1u l=180n
M298 t123 t118 0 0 nch w=1u l=180n
M299 nw27 t119 vdd vdd pch w=2u l=180n
M300 nw27 t120 vdd vdd pch w=2u l=180n
CT124 t124 0 0.1f
M301 nw27 t119 t124 0 nch w=1u l=180n
M302 t124 t120 0 0 nch w=1u l=180n
Cnw27 nw27 0 2f
CT125 t125 0 0.1f
M303 t125 nw26 vdd vdd pch w=2u l=180n
M304 t125 nq13 vdd vdd pch w=2u l=180n
CT126 t126 0 0.1f
M305 t125 nw26 t126 0 nch w=1u l=180n
M306 t126 nq13 0 0 nch w=1u l=180n
M307 nw28 t125 vdd vdd pch w=2u l=180n
M308 nw28 t125 0 0 nch w=1u l=180n
Cnw28 nw28 0 2f
CT127 t127 0 0.1f
CT128 t128 0 0.1f
CT129 t129 0 0.1f
M309 t127 nq14 vdd vdd pch w=2u l=180n
M310 t127 nw28 vdd vdd pch w=2u l=180n
CT130 t130 0 0.1f
M311 t127 nq14 t130 0 nch w=1u l=180n
M312 t130 nw28 0 0 nch w=1u l=180n
M313 t128 nq14 vdd vdd pch w=2u l=180n
M314 t128 t127 vdd vdd pch w=2u l=180n
CT131 t131 0 0.1f
M315 t128 nq14 t131 0 nch w=1u l=180n
M316 t131 t127 0 0 nch w=1u l=180n
M317 t129 nw28 vdd vdd pch w=2u l=180n
M318 t129 t127 vdd vdd pch w=2u l=180n
CT132 t132 0 0.1f
M319 t129 nw28 t132 0 nch w=1u l=180n
M320 t132 t127 0 0 nch w=1u l=180n
M321 nw29 t128 vdd vdd pch w=2u l=180n
M322 nw29 t129 vdd vdd pch w=2u l=180n
CT133 t133 0 0.1f
M323 nw29 t128 t133 0 nch w=1u l=180n
M324 t133 t129 0 0 nch w=1u l=180n
Cnw29 nw29 0 2f
CT134 t134 0 0.1f
M325 t134 nw28 vdd vdd pch w=2u l=180n
M326 t134 nq14 vdd vdd pch w=2u l=180n
CT135 t135 0 0.1f
M327 t134 nw28 t135 0 nch w=1u l=180n
M328 t135 nq14 0 0 nch w=1u l=180n
M329 nw30 t134 vdd vdd pch w=2u l=180n
M330 nw30 t134 0 0 nch w=1u l=180n
Cnw30 nw30 0 2f
CT136 t136 0 0.1f
CT137 t137 0 0.1f
CT138 t138 0 0.1f
M331 t136 nq15 vdd vdd pch w=2u l=180n
M332 t136 nw30 vdd vdd pch w=2u l=180n
CT139 t139 0 0.1f
M333 t136 nq15 t139 0 nch w=1u l=180n
M334 t139 nw30 0 0 nch w=1u l=180n
M335 t137 nq15 vdd vdd pch w=2u l=180n
M336 t137 t136 vdd vdd pch w=2u l=180n
CT140 t140 0 0.1f
M337 t137 nq15 t140 0 nch w=1u l=180n
M338 t140 t136 0 0 nch w=1u l=180n
M339 t138 nw30 vdd vdd pch w=2u l=180n
M340 t138 t136 vdd vdd pch w=2u l=180n
CT141 t141 0 0.1f
M341 t138 nw30 t141 0 nch w=1u l=180n
M342 t141 t136 0 0 nch w=1u l=180n
M343 nw31 t137 vdd vdd pch w=2u l=180n
M344 nw31 t138 vdd vdd pch w=2u l=180n
CT142 t142 0 0.1f
M345 nw31 t137 t142 0 nch w=1u l=180n
M346 t142 t138 0 0 nch w=1u l=180n
Cnw31 nw31 0 2f
CT143 t143 0 0.1f
M347 t143 nw30 vdd vdd pch w=2u l=180n
M348 t143 nq15 vdd vdd pch w=2u l=180n
CT144 t144 0 0.1f
M349 t143 nw30 t144 0 nch w=1u l=180n
M350 t144 nq15 0 0 nch w=1u l=180n
M351 nw32 t143 vdd vdd pch w=2u l=180n
M352 nw32 t143 0 0 nch w=1u l=180n
Cnw32 nw32 0 2f
CT145 t145 0 0.1f
CT146 t146 0 0.1f
CT147 t147 0 0.1f
M353 t145 nq16 vdd vdd pch w=2u l=180n
M354 t145 nw32 vdd vdd pch w=2u l=180n
CT148 t148 0 0.1f
M355 t145 nq16 t148 0 nch w=1u l=180n
M356 t148 nw32 0 0 nch w=1u l=180n
M357 t146 nq16 vdd vdd pch w=2u l=180n
M358 t146 t145 vdd vdd pch w=2u l=180n
CT149 t149 0 0.1f
M359 t146 nq16 t149 0 nch w=1u l=180n
M360 t149 t145 0 0 nch w=1u l=180n
M361 t147 nw32 vdd vdd pch w=2u l=180n
M362 t147 t145 vdd vdd pch w=2u l=180n
CT150 t150 0 0.1f
M363 t147 nw32 t150 0 nch w=1u l=180n
M364 t150 t145 0 0 nch w=1u l=180n
M365 nw33 t146 vdd vdd pch w=2u l=180n
M366 nw33 t147 vdd vdd pch w=2u l=180n
CT151 t151 0 0.1f
M367 nw33 t146 t151 0 nch w=1u l=180n
M368 t151 t147 0 0 nch w=1u l=180n
Cnw33 nw33 0 2f
CT152 t152 0 0.1f
M369 t152 nw32 vdd vdd pch w=2u l=180n
M370 t152 nq16 vdd vdd pch w=2u l=180n
CT153 t153 0 0.1f
M371 t152 nw32 t153 0 nch w=1u l=180n
M372 t153 nq16 0 0 nch w=1u l=180n
M373 nw34 t152 vdd vdd pch w=2u l=180n
M374 nw34 t152 0 0 nch w=1u l=180n
Cnw34 nw34 0 2f
CT154 t154 0 0.1f
CT155 t155 0 0.1f
CT156 t156 0 0.1f
M375 t154 nq17 vdd vdd pch w=2u l=180n
M376 t154 nw34 vdd vdd pch w=2u l=180n
CT157 t157 0 0.1f
M377 t154 nq17 t157 0 nch w=1u l=180n
M378 t157 nw34 0 0 nch w=1u l=180n
M379 t155 nq17 vdd vdd pch w=2u l=180n
M380 t155 t154 vdd vdd pch w=2u l=180n
CT158 t158 0 0.1f
M381 t155 nq17 t158 0 nch w=1u l=180n
M382 t158 t154 0 0 nch w=1u l=180n
M383 t156 nw34 vdd vdd pch w=2u l=180n
M384 t156 t154 vdd vdd pch w=2u l=180n
CT159 t159 0 0.1f
M385 t156 nw34 t159 0 nch w=1u l=180n
M386 t159 t154 0 0 nch w=1u l=180n
M387 nw35 t155 vdd vdd pch w=2u l=180n
M388 nw35 t156 vdd vdd pch w=2u l=180n
CT160 t160 0 0.1f
M389 nw35 t155 t160 0 nch w=1u l=180n
M390 t160 t156 0 0 nch w=1u l=180n
Cnw35 nw35 0 2f
CT161 t161 0 0.1f
M391 t161 nw34 vdd vdd pch w=2u l=180n
M392 t161 nq17 vdd vdd pch w=2u l=180n
CT162 t162 0 0.1f
M393 t161 nw34 t162 0 nch w=1u l=180n
M394 t162 nq17 0 0 nch w=1u l=180n
M395 nw36 t161 vdd vdd pch w=2u l=180n
M396 nw36 t161 0 0 nch w=1u l=180n
Cnw36 nw36 0 2f
CT163 t163 0 0.1f
CT164 t164 0 0.1f
CT165 t165 0 0.1f
M397 t163 nq18 vdd vdd pch w=2u l=180n
M398 t163 nw36 vdd vdd pch w=2u l=180n
CT166 t166 0 0.1f
M399 t163 nq18 t166 0 nch w=1u l=180n
M400 t166 nw36 0 0 nch w=1u l=180n
M401 t164 nq18 vdd vdd pch w=2u l=180n
M402 t164 t163 vdd vdd pch w=2u l=180n
CT167 t167 0 0.1f
M403 t164 nq18 t167 0 nch w=1u l=180n
M404 t167 t163 0 0 nch w=1u l=180n
M405 t165 nw36 vdd vdd pch w=2u l=180n
M406 t165 t163 vdd vdd pch w=2u l=180n
CT168 t168 0 0.1f
M407 t165 nw36 t168 0 nch w=1u l=180n
M408 t168 t163 0 0 nch w=1u l=180n
M409 nw37 t164 vdd vdd pch w=2u l=180n
M410 nw37 t165 vdd vdd pch w=2u l=180n
CT169 t169 0 0.1f
M411 nw37 t164 t169 0 nch w=1u l=180n
M412 t169 t165 0 0 nch w=1u l=180n
Cnw37 nw37 0 2f
CT170 t170 0 0.1f
M413 t170 nw36 vdd vdd pch w=2u l=180n
M414 t170 nq18 vdd vdd pch w=2u l=180n
CT171 t171 0 0.1f
M415 t170 nw36 t171 0 nch w=1u l=180n
M416 t171 nq18 0 0 nch w=1u l=180n
M417 nw38 t170 vdd vdd pch w=2u l=180n
M418 nw38 t170 0 0 nch w=1u l=180n
Cnw38 nw38 0 2f
CT172 t172 0 0.1f
CT173 t173 0 0.1f
CT174 t174 0 0.1f
M419 t172 nq19 vdd vdd pch w=2u l=180n
M420 t172 nw38 vdd vdd pch w=2u l=180n
CT175 t175 0 0.1f
M421 t172 nq19 t175 0 nch w=1u l=180n
M422 t175 nw38 0 0 nch w=1u l=180n
M423 t173 nq19 vdd vdd pch w=2u l=180n
M424 t173 t172 vdd vdd pch w=2u l=180n
CT176 t176 0 0.1f
M425 t173 nq19 t176 0 nch w=1u l=180n
M426 t176 t172 0 0 nch w=1u l=180n
M427 t174 nw38 vdd vdd pch w=2u l=180n
M428 t174 t172 vdd vdd pch w=2u l=180n
CT177 t177 0 0.1f
M429 t174 nw38 t177 0 nch w=1u l=180n
M430 t177 t172 0 0 nch w=1u l=180n
M431 nw39 t173 vdd vdd pch w=2u l=180n
M432 nw39 t174 vdd vdd pch w=2u l=180n
CT178 t178 0 0.1f
M433 nw39 t173 t178 0 nch w=1u l=180n
M434 t178 t174 0 0 nch w=1u l=180n
Cnw39 nw39 0 2f
CT179 t179 0 0.1f
M435 t179 nw38 vdd vdd pch w=2u l=180n
M436 t179 nq19 vdd vdd pch w=2u l=180n
CT180 t180 0 0.1f
M437 t179 nw38 t180 0 nch w=1u l=180n
M438 t180 nq19 0 0 nch w=1u l=180n
M439 nw40 t179 vdd vdd pch w=2u l=180n
M440 nw40 t179 0 0 nch w=1u l=180n
Cnw40 nw40 0 2f
CT181 t181 0 0.1f
CT182 t182 0 0.1f
CT183 t183 0 0.1f
M441 t181 nq20 vdd vdd pch w=2u l=180n
M442 t181 nw40 vdd vdd pch w=2u l=180n
CT184 t184 0 0.1f
M443 t181 nq20 t184 0 nch w=1u l=180n
M444 t184 nw40 0 0 nch w=1u l=180n
M445 t182 nq20 vdd vdd pch w=2u l=180n
M446 t182 t181 vdd vdd pch w=2u l=180n
CT185 t185 0 0.1f
M447 t182 nq20 t185 0 nch w=1u l=180n
M448 t185 t181 0 0 nch w=1u l=180n
M449 t183 nw40 vdd vdd pch w=2u l=180n
M450 t183 t181 vdd vdd pch w=2u l=180n
CT186 t186 0 0.1f
M451 t183 nw40 t186 0 nch w=1u l=180n
M452 t186 t181 0 0 nch w=1u l=180n
M453 nw41 t182 vdd vdd pch w=2u l=180n
M454 nw41 t183 vdd vdd pch w=2u l=180n
CT187 t187 0 0.1f
M455 nw41 t182 t187 0 nch w=1u l=180n
M456 t187 t183 0 0 nch w=1u l=180n
Cnw41 nw41 0 2f
CT188 t188 0 0.1f
M457 t188 nw40 vdd vdd pch w=2u l=180n
M458 t188 nq20 vdd vdd pch w=2u l=180n
CT189 t189 0 0.1f
M459 t188 nw40 t189 0 nch w=1u l=180n
M460 t189 nq20 0 0 nch w=1u l=180n
M461 nw42 t188 vdd vdd pch w=2u l=180n
M462 nw42 t188 0 0 nch w=1u l=180n
Cnw42 nw42 0 2f
CT190 t190 0 0.1f
CT191 t191 0 0.1f
CT192 t192 0 0.1f
M463 t190 nq21 vdd vdd pch w=2u l=180n
M464 t190 nw42 vdd vdd pch w=2u l=180n
CT193 t193 0 0.1f
M465 t190 nq21 t193 0 nch w=1u l=180n
M466 t193 nw42 0 0 nch w=1u l=180n
M467 t191 nq21 vdd vdd pch w=2u l=180n
M468 t191 t190 vdd vdd pch w=2u l=180n
CT194 t194 0 0.1f
M469 t191 nq21 t194 0 nch w=1u l=180n
M470 t194 t190 0 0 nch w=1u l=180n
M471 t192 nw42 vdd vdd pch w=2u l=180n
M472 t192 t190 vdd vdd pch w=2u l=180n
CT195 t195 0 0.1f
M473 t192 nw42 t195 0 nch w=1u l=180n
M474 t195 t190 0 0 nch w=1u l=180n
M475 nw43 t191 vdd vdd pch w=2u l=180n
M476 nw43 t192 vdd vdd pch w=2u l=180n
CT196 t196 0 0.1f
M477 nw43 t191 t196 0 nch w=1u l=180n
M478 t196 t192 0 0 nch w=1u l=180n
Cnw43 nw43 0 2f
CT197 t197 0 0.1f
M479 t197 nw42 vdd vdd pch w=2u l=180n
M480 t197 nq21 vdd vdd pch w=2u l=180n
CT198 t198 0 0.1f
M481 t197 nw42 t198 0 nch w=1u l=180n
M482 t198 nq21 0 0 nch w=1u l=180n
M483 nw44 t197 vdd vdd pch w=2u l=180n
M484 nw44 t197 0 0 nch w=1u l=180n
Cnw44 nw44 0 2f
CT199 t199 0 0.1f
CT200 t200 0 0.1f
CT201 t201 0 0.1f
M485 t199 nq22 vdd vdd pch w=2u l=180n
M486 t199 nw44 vdd vdd pch w=2u l=180n
CT202 t202 0 0.1f
M487 t199 nq22 t202 0 nch w=1u l=180n
M488 t202 nw44 0 0 nch w=1u l=180n
M489 t200 nq22 vdd vdd pch w=2u l=180n
M490 t200 t199 vdd vdd pch w=2u l=180n
CT203 t203 0 0.1f
M491 t200 nq22 t203 0 nch w=1u l=180n
M492 t203 t199 0 0 nch w=1u l=180n
M493 t201 nw44 vdd vdd pch w=2u l=180n
M494 t201 t199 vdd vdd pch w=2u l=180n
CT204 t204 0 0.1f
M495 t201 nw44 t204 0 nch w=1u l=180n
M496 t204 t199 0 0 nch w=1u l=180n
M497 nw45 t200 vdd vdd pch w=2u l=180n
M498 nw45 t201 vdd vdd pch w=2u l=180n
CT205 t205 0 0.1f
M499 nw45 t200 t205 0 nch w=1u l=180n
M500 t205 t201 0 0 nch w=1u l=180n
Cnw45 nw45 0 2f
CT206 t206 0 0.1f
M501 t206 nw44 vdd vdd pch w=2u l=180n
M502 t206 nq22 vdd vdd pch w=2u l=180n
CT207 t207 0 0.1f
M503 t206 nw44 t207 0 nch w=1u l=180n
M504 t207 nq22 0 0 nch w=1u l=180n
M505 nw46 t206 vdd vdd pch w=2u l=180n
M506 nw46 t206 0 0 nch w=1u l=180n
Cnw46 nw46 0 2f
CT208 t208 0 0.1f
CT209 t209 0 0.1f
CT210 t210 0 0.1f
M507 t208 nq23 vdd vdd pch w=2u l=180n
M508 t208 nw46 vdd vdd pch w=2u l=180n
CT211 t211 0 0.1f
M509 t208 nq23 t211 0 nch w=1u l=180n
M510 t211 nw46 0 0 nch w=1u l=180n
M511 t209 nq23 vdd vdd pch w=2u l=180n
M512 t209 t208 vdd vdd pch w=2u l=180n
CT212 t212 0 0.1f
M513 t209 nq23 t212 0 nch w=1u l=180n
M514 t212 t208 0 0 nch w=1u l=180n
M515 t210 nw46 vdd vdd pch w=2u l=180n
M516 t210 t208 vdd vdd pch w=2u l=180n
CT213 t213 0 0.1f
M517 t210 nw46 t213 0 nch w=1u l=180n
M518 t213 t208 0 0 nch w=1u l=180n
M519 nw47 t209 vdd vdd pch w=2u l=180n
M520 nw47 t210 vdd vdd pch w=2u l=180n
CT214 t214 0 0.1f
M521 nw47 t209 t214 0 nch w=1u l=180n
M522 t214 t210 0 0 nch w=1u l=180n
Cnw47 nw47 0 2f
CT215 t215 0 0.1f
M523 t215 nw46 vdd vdd pch w=2u l=180n
M524 t215 nq23 vdd vdd pch w=2u l=180n
CT216 t216 0 0.1f
M525 t215 nw46 t216 0 nch w=1u l=180n
M526 t216 nq23 0 0 nch w=1u l=180n
M527 nw48 t215 vdd vdd pch w=2u l=180n
M528 nw48 t215 0 0 nch w=1u l=180n
Cnw48 nw48 0 2f
CT217 t217 0 0.1f
CT218 t218 0 0.1f
CT219 t219 0 0.1f
M529 t217 nq24 vdd vdd pch w=2u l=180n
M530 t217 nw48 vdd vdd pch w=2u l=180n
CT220 t220 0 0.1f
M531 t217 nq24 t220 0 nch w=1u l=180n
M532 t220 nw48 0 0 nch w=1u l=180n
M533 t218 nq24 vdd vdd pch w=2u l=180n
M534 t218 t217 vdd vdd pch w=2u l=180n
CT221 t221 0 0.1f
M535 t218 nq24 t221 0 nch w=1u l=180n
M536 t221 t217 0 0 nch w=1u l=180n
M537 t219 nw48 vdd vdd pch w=2u l=180n
M538 t219 t217 vdd vdd pch w=2u l=180n
CT222 t222 0 0.1f
M539 t219 nw48 t222 0 nch w=1u l=180n
M540 t222 t217 0 0 nch w=1u l=180n
M541 nw49 t218 vdd vdd pch w=2u l=180n
M542 nw49 t219 vdd vdd pch w=2u l=180n
CT223 t223 0 0.1f
M543 nw49 t218 t223 0 nch w=1u l=180n
M544 t223 t219 0 0 nch w=1u l=180n
Cnw49 nw49 0 2f
CT224 t224 0 0.1f
M545 t224 nw48 vdd vdd pch w=2u l=180n
M546 t224 nq24 vdd vdd pch w=2u l=180n
CT225 t225 0 0.1f
M547 t224 nw48 t225 0 nch w=1u l=180n
M548 t225 nq24 0 0 nch w=1u l=180n
M549 nw50 t224 vdd vdd pch w=2u l=180n
M550 nw50 t224 0 0 nch w=1u l=180n
Cnw50 nw50 0 2f
CT226 t226 0 0.1f
CT227 t227 0 0.1f
CT228 t228 0 0.1f
M551 t226 nq25 vdd vdd pch w=2u l=180n
M552 t226 nw50 vdd vdd pch w=2u l=180n
CT229 t229 0 0.1f
M553 t226 nq25 t229 0 nch w=1u l=180n
M554 t229 nw50 0 0 nch w=1u l=180n
M555 t227 nq25 vdd vdd pch w=2u l=180n
M556 t227 t226 vdd vdd pch w=2u l=180n
CT230 t230 0 0.1f
M557 t227 nq25 t230 0 nch w=1u l=180n
M558 t230 t226 0 0 nch w=1u l=180n
M559 t228 nw50 vdd vdd pch w=2u l=180n
M560 t228 t226 vdd vdd pch w=2u l=180n
CT231 t231 0 0.1f
M561 t228 nw50 t231 0 nch w=1u l=180n
M562 t231 t226 0 0 nch w=1u l=180n
M563 nw51 t227 vdd vdd pch w=2u l=180n
M564 nw51 t228 vdd vdd pch w=2u l=180n
CT232 t232 0 0.1f
M565 nw51 t227 t232 0 nch w=1u l=180n
M566 t232 t228 0 0 nch w=1u l=180n
Cnw51 nw51 0 2f
CT233 t233 0 0.1f
M567 t233 nw50 vdd vdd pch w=2u l=180n
M568 t233 nq25 vdd vdd pch w=2u l=180n
CT234 t234 0 0.1f
M569 t233 nw50 t234 0 nch w=1u l=180n
M570 t234 nq25 0 0 nch w=1u l=180n
M571 nw52 t233 vdd vdd pch w=2u l=180n
M572 nw52 t233 0 0 nch w=1u l=180n
Cnw52 nw52 0 2f
CT235 t235 0 0.1f
CT236 t236 0 0.1f
CT237 t237 0 0.1f
M573 t235 nq26 vdd vdd pch w=2u l=180n
M574 t235 nw52 vdd vdd pch w=2u l=180n
CT238 t238 0 0.1f
M575 t235 nq26 t238 0 nch w=1u l=180n
M576 t238 nw52 0 0 nch w=1u l=180n
M577 t236 nq26 vdd vdd pch w=2u l=180n
M578 t236 t235 vdd vdd pch w=2u l=180n
CT239 t239 0 0.1f
M579 t236 nq26 t239 0 nch w=1u l=180n
M580 t239 t235 0 0 nch w=1u l=180n
M581 t237 nw52 vdd vdd pch w=2u l=180n
M582 t237 t235 vdd vdd pch w=2u l=180n
CT240 t240 0 0.1f
M583 t237 nw52 t240 0 nch w=1u l=180n
M584 t240 t235 0 0 nch w=1u l=180n
M585 nw53 t236 vdd vdd pch w=2u l=180n
M586 nw53 t237 vdd vdd pch w=2u l=180n
CT241 t241 0 0.1f
M587 nw53 t236 t241 0 nch w=1u l=180n
M588 t241 t237 0 0 nch w=1u l=180n
Cnw53 nw53 0 2f
CT242 t242 0 0.1f
M589 t242 nw52 vdd vdd pch w=2u l=180n
M590 t242 nq26 vdd vdd pch w=2u l=180n
CT243 t243 0 0.1f
M591 t242 nw52 t243 0 nch w=1u l=180n
M592 t243 nq26 0 0 nch w=1u l=180n
M593 nw54 t242 vdd vdd pch w=2u l=180n
M594 nw54 t242 0 0 nch w=1u l=180n
Cnw54 nw54 0 2f
CT244 t244 0 0.1f
CT245 t245 0 0.1f
CT246 t246 0 0.1f
M595 t244 nq27 vdd vdd pch w=2u l=180n
M596 t244 nw54 vdd vdd pch w=2u l=180n
CT247 t247 0 0.1f
M597 t244 nq27 t247 0 nch w=1u l=180n
M598 t247 nw54 0 0 nch w=1u l=180n
M599 t245 nq27 vdd vdd pch w=2u l=180n
M600 t245 t244 vdd vdd pch w=2u l=180n
CT248 t248 0 0.1f
M601 t245 nq27 t248 0 nch w=1u l=180n
M602 t248 t244 0 0 nch w=1u l=180n
M603 t246 nw54 vdd vdd pch w=2u l=180n
M604 t246 t244 vdd vdd pch w=2u l=180n
CT249 t249 0 0.1f
M605 t246 nw54 t249 0 nch w=1u l=180n
M606 t249 t244 0 0 nch w=1u l=180n
M607 nw55 t245 vdd vdd pch w=2u l=180n
M608 nw55 t246 vdd vdd pch w=2u l=180n
CT250 t250 0 0.1f
M609 nw55 t245 t250 0 nch w=1u l=180n
M610 t250 t246 0 0 nch w=1u l=180n
Cnw55 nw55 0 2f
CT251 t251 0 0.1f
M611 t251 nw54 vdd vdd pch w=2u l=180n
M612 t251 nq27 vdd vdd pch w=2u l=180n
CT252 t252 0 0.1f
M613 t251 nw54 t252 0 nch w=1u l=180n
M614 t252 nq27 0 0 nch w=1u l=180n
M615 nw56 t251 vdd vdd pch w=2u l=180n
M616 nw56 t251 0 0 nch w=1u l=180n
Cnw56 nw56 0 2f
CT253 t253 0 0.1f
CT254 t254 0 0.1f
CT255 t255 0 0.1f
M617 t253 nq28 vdd vdd pch w=2u l=180n
M618 t253 nw56 vdd vdd pch w=2u l=180n
CT256 t256 0 0.1f
M619 t253 nq28 t256 0 nch w=1u l=180n
M620 t256 nw56 0 0 nch w=1u l=180n
M621 t254 nq28 vdd vdd pch w=2u l=180n
M622 t254 t253 vdd vdd pch w=2u l=180n
CT257 t257 0 0.1f
M623 t254 nq28 t257 0 nch w=1u l=180n
M624 t257 t253 0 0 nch w=1u l=180n
M625 t255 nw56 vdd vdd pch w=2u l=180n
M626 t255 t253 vdd vdd pch w=2u l=180n
CT258 t258 0 0.1f
M627 t255 nw56 t258 0 nch w=1u l=180n
M628 t258 t253 0 0 nch w=1u l=180n
M629 nw57 t254 vdd vdd pch w=2u l=180n
M630 nw57 t255 vdd vdd pch w=2u l=180n
CT259 t259 0 0.1f
M631 nw57 t254 t259 0 nch w=1u l=180n
M632 t259 t255 0 0 nch w=1u l=180n
Cnw57 nw57 0 2f
CT260 t260 0 0.1f
M633 t260 nw56 vdd vdd pch w=2u l=180n
M634 t260 nq28 vdd vdd pch w=2u l=180n
CT261 t261 0 0.1f
M635 t260 nw56 t261 0 nch w=1u l=180n
M636 t261 nq28 0 0 nch w=1u l=180n
M637 nw58 t260 vdd vdd pch w=2u l=180n
M638 nw58 t260 0 0 nch w=1u l=180n
Cnw58 nw58 0 2f
CT262 t262 0 0.1f
CT263 t263 0 0.1f
CT264 t264 0 0.1f
M639 t262 nq29 vdd vdd pch w=2u l=180n
M640 t262 nw58 vdd vdd pch w=2u l=180n
CT265 t265 0 0.1f
M641 t262 nq29 t265 0 nch w=1u l=180n
M642 t265 nw58 0 0 nch w=1u l=180n
M643 t263 nq29 vdd vdd pch w=2u l=180n
M644 t263 t262 vdd vdd pch w=2u l=180n
CT266 t266 0 0.1f
M645 t263 nq29 t266 0 nch w=1u l=180n
M646 t266 t262 0 0 nch w=1u l=180n
M647 t264 nw58 vdd vdd pch w=2u l=180n
M648 t264 t262 vdd vdd pch w=2u l=180n
CT267 t267 0 0.1f
M649 t264 nw58 t267 0 nch w=1u l=180n
M650 t267 t262 0 0 nch w=1u l=180n
M651 nw59 t263 vdd vdd pch w=2u l=180n
M652 nw59 t264 vdd vdd pch w=2u l=180n
CT268 t268 0 0.1f
M653 nw59 t263 t268 0 nch w=1u l=180n
M654 t268 t264 0 0 nch w=1u l=180n
Cnw59 nw59 0 2f
CT269 t269 0 0.1f
M655 t269 nw58 vdd vdd pch w=2u l=180n
M656 t269 nq29 vdd vdd pch w=2u l=180n
CT270 t270 0 0.1f
M657 t269 nw58 t270 0 nch w=1u l=180n
M658 t270 nq29 0 0 nch w=1u l=180n
M659 nw60 t269 vdd vdd pch w=2u l=180n
M660 nw60 t269 0 0 nch w=1u l=180n
Cnw60 nw60 0 2f
CT271 t271 0 0.1f
CT272 t272 0 0.1f
CT273 t273 0 0.1f
M661 t271 nq30 vdd vdd pch w=2u l=180n
M662 t271 nw60 vdd vdd pch w=2u l=180n
CT274 t274 0 0.1f
M663 t271 nq30 t274 0 nch w=1u l=180n
M664 t274 nw60 0 0 nch w=1u l=180n
M665 t272 nq30 vdd vdd pch w=2u l=180n
M666 t272 t271 vdd vdd pch w=2u l=180n
CT275 t275 0 0.1f
M667 t272 nq30 t275 0 nch w=1u l=180n
M668 t275 t271 0 0 nch w=1u l=180n
M669 t273 nw60 vdd vdd pch w=2u l=180n
M670 t273 t271 vdd vdd pch w=2u l=180n
CT276 t276 0 0.1f
M671 t273 nw60 t276 0 nch w=1u l=180n
M672 t276 t271 0 0 nch w=1u l=180n
M673 nw61 t272 vdd vdd pch w=2u l=180n
M674 nw61 t273 vdd vdd pch w=2u l=180n
CT277 t277 0 0.1f
M675 nw61 t272 t277 0 nch w=1u l=180n
M676 t277 t273 0 0 nch w=1u l=180n
Cnw61 nw61 0 2f
CT278 t278 0 0.1f
M677 t278 nw60 vdd vdd pch w=2u l=180n
M678 t278 nq30 vdd vdd pch w=2u l=180n
CT279 t279 0 0.1f
M679 t278 nw60 t279 0 nch w=1u l=180n
M680 t279 nq30 0 0 nch w=1u l=180n
M681 nw62 t278 vdd vdd pch w=2u l=180n
M682 nw62 t278 0 0 nch w=1u l=180n
Cnw62 nw62 0 2f
CT280 t280 0 0.1f
CT281 t281 0 0.1f
CT282 t282 0 0.1f
M683 t280 nq31 vdd vdd pch w=2u l=180n
M684 t280 nw62 vdd vdd pch w=2u l=180n
CT283 t283 0 0.1f
M685 t280 nq31 t283 0 nch w=1u l=180n
M686 t283 nw62 0 0 nch w=1u l=180n
M687 t281 nq31 vdd vdd pch w=2u l=180n
M688 t281 t280 vdd vdd pch w=2u l=180n
CT284 t284 0 0.1f
M689 t281 nq31 t284 0 nch w=1u l=180n
M690 t284 t280 0 0 nch w=1u l=180n
M691 t282 nw62 vdd vdd pch w=2u l=180n
M692 t282 t280 vdd vdd pch w=2u l=180n
CT285 t285 0 0.1f
M693 t282 nw62 t285 0 nch w=1u l=180n
M694 t285 t280 0 0 nch w=1u l=180n
M695 nw63 t281 vdd vdd pch w=2u l=180n
M696 nw63 t282 vdd vdd pch w=2u l=180n
CT286 t286 0 0.1f
M697 nw63 t281 t286 0 nch w=1u l=180n
M698 t286 t282 0 0 nch w=1u l=180n
Cnw63 nw63 0 2f
CT287 t287 0 0.1f
M699 t287 nw62 vdd vdd pch w=2u l=180n
M700 t287 nq31 vdd vdd pch w=2u l=180n
CT288 t288 0 0.1f
M701 t287 nw62 t288 0 nch w=1u l=180n
M702 t288 nq31 0 0 nch w=1u l=180n
M703 nw64 t287 vdd vdd pch w=2u l=180n
M704 nw64 t287 0 0 nch w=1u l=180n
Cnw64 nw64 0 2f
CT289 t289 0 0.1f
CT290 t290 0 0.1f
CT291 t291 0 0.1f
M705 t289 nq32 vdd vdd pch w=2u l=180n
M706 t289 nw64 vdd vdd pch w=2u l=180n
CT292 t292 0 0.1f
M707 t289 nq32 t292 0 nch w=1u l=180n
M708 t292 nw64 0 0 nch w=1u l=180n
M709 t290 nq32 vdd vdd pch w=2u l=180n
M710 t290 t289 vdd vdd pch w=2u l=180n
CT293 t293 0 0.1f
M711 t290 nq32 t293 0 nch w=1u l=180n
M712 t293 t289 0 0 nch w=1u l=180n
M713 t291 nw64 vdd vdd pch w=2u l=180n
M714 t291 t289 vdd vdd pch w=2u l=180n
CT294 t294 0 0.1f
M715 t291 nw64 t294 0 nch w=1u l=180n
M716 t294 t289 0 0 nch w=1u l=180n
M717 nw65 t290 vdd vdd pch w=2u l=180n
M718 nw65 t291 vdd vdd pch w=2u l=180n
CT295 t295 0 0.1f
M719 nw65 t290 t295 0 nch w=1u l=180n
M720 t295 t291 0 0 nch w=1u l=180n
Cnw65 nw65 0 2f
CT296 t296 0 0.1f
M721 t296 nw64 vdd vdd pch w=2u l=180n
M722 t296 nq32 vdd vdd pch w=2u l=180n
CT297 t297 0 0.1f
M723 t296 nw64 t297 0 nch w=1u l=180n
M724 t297 nq32 0 0 nch w=1u l=180n
M725 nw66 t296 vdd vdd pch w=2u l=180n
M726 nw66 t296 0 0 nch w=1u l=180n
Cnw66 nw66 0 2f
CT298 t298 0 0.1f
CT299 t299 0 0.1f
CT300 t300 0 0.1f
M727 t298 nq33 vdd vdd pch w=2u l=180n
M728 t298 nw66 vdd vdd pch w=2u l=180n
CT301 t301 0 0.1f
M729 t298 nq33 t301 0 nch w=1u l=180n
M730 t301 nw66 0 0 nch w=1u l=180n
M731 t299 nq33 vdd vdd pch w=2u l=180n
M732 t299 t298 vdd vdd pch w=2u l=180n
CT302 t302 0 0.1f
M733 t299 nq33 t302 0 nch w=1u l=180n
M734 t302 t298 0 0 nch w=1u l=180n
M735 t300 nw66 vdd vdd pch w=2u l=180n
M736 t300 t298 vdd vdd pch w=2u l=180n
CT303 t303 0 0.1f
M737 t300 nw66 t303 0 nch w=1u l=180n
M738 t303 t298 0 0 nch w=1u l=180n
M739 nw67 t299 vdd vdd pch w=2u l=180n
M740 nw67 t300 vdd vdd pch w=2u l=180n
CT304 t304 0 0.1f
M741 nw67 t299 t304 0 nch w=1u l=180n
M742 t304 t300 0 0 nch w=1u l=180n
Cnw67 nw67 0 2f
CT305 t305 0 0.1f
M743 t305 nw66 vdd vdd pch w=2u l=180n
M744 t305 nq33 vdd vdd pch w=2u l=180n
CT306 t306 0 0.1f
M745 t305 nw66 t306 0 nch w=1u l=180n
M746 t306 nq33 0 0 nch w=1u l=180n
M747 nw68 t305 vdd vdd pch w=2u l=180n
M748 nw68 t305 0 0 nch w=1u l=180n
Cnw68 nw68 0 2f
CT307 t307 0 0.1f
CT308 t308 0 0.1f
CT309 t309 0 0.1f
M749 t307 nq34 vdd vdd pch w=2u l=180n
M750 t307 nw68 vdd vdd pch w=2u l=180n
CT310 t310 0 0.1f
M751 t307 nq34 t310 0 nch w=1u l=180n
M752 t310 nw68 0 0 nch w=1u l=180n
M753 t308 nq34 vdd vdd pch w=2u l=180n
M754 t308 t307 vdd vdd pch w=2u l=180n
CT311 t311 0 0.1f
M755 t308 nq34 t311 0 nch w=1u l=180n
M756 t311 t307 0 0 nch w=1u l=180n
M757 t309 nw68 vdd vdd pch w=2u l=180n
M758 t309 t307 vdd vdd pch w=2u l=180n
CT312 t312 0 0.1f
M759 t309 nw68 t312 0 nch w=1u l=180n
M760 t312 t307 0 0 nch w=1u l=180n
M761 nw69 t308 vdd vdd pch w=2u l=180n
M762 nw69 t309 vdd vdd pch w=2u l=180n
CT313 t313 0 0.1f
M763 nw69 t308 t313 0 nch w=1u l=180n
M764 t313 t309 0 0 nch w=1u l=180n
Cnw69 nw69 0 2f
CT314 t314 0 0.1f
M765 t314 nw68 vdd vdd pch w=2u l=180n
M766 t314 nq34 vdd vdd pch w=2u l=180n
CT315 t315 0 0.1f
M767 t314 nw68 t315 0 nch w=1u l=180n
M768 t315 nq34 0 0 nch w=1u l=180n
M769 nw70 t314 vdd vdd pch w=2u l=180n
M770 nw70 t314 0 0 nch w=1u l=180n
Cnw70 nw70 0 2f
CT316 t316 0 0.1f
CT317 t317 0 0.1f
CT318 t318 0 0.1f
M771 t316 nq35 vdd vdd pch w=2u l=180n
M772 t316 nw70 vdd vdd pch w=2u l=180n
CT319 t319 0 0.1f
M773 t316 nq35 t319 0 nch w=1u l=180n
M774 t319 nw70 0 0 nch w=1u l=180n
M775 t317 nq35 vdd vdd pch w=2u l=180n
M776 t317 t316 vdd vdd pch w=2u l=180n
CT320 t320 0 0.1f
M777 t317 nq35 t320 0 nch w=1u l=180n
M778 t320 t316 0 0 nch w=1u l=180n
M779 t318 nw70 vdd vdd pch w=2u l=180n
M780 t318 t316 vdd vdd pch w=2u l=180n
CT321 t321 0 0.1f
M781 t318 nw70 t321 0 nch w=1u l=180n
M782 t321 t316 0 0 nch w=1u l=180n
M783 nw71 t317 vdd vdd pch w=2u l=180n
M784 nw71 t318 vdd vdd pch w=2u l=180n
CT322 t322 0 0.1f
M785 nw71 t317 t322 0 nch w=1u l=180n
M786 t322 t318 0 0 nch w=1u l=180n
Cnw71 nw71 0 2f
CT323 t323 0 0.1f
M787 t323 nw70 vdd vdd pch w=2u l=180n
M788 t323 nq35 vdd vdd pch w=2u l=180n
CT324 t324 0 0.1f
M789 t323 nw70 t324 0 nch w=1u l=180n
M790 t324 nq35 0 0 nch w=1u l=180n
M791 nw72 t323 vdd vdd pch w=2u l=180n
M792 nw72 t323 0 0 nch w=1u l=180n
Cnw72 nw72 0 2f
CT325 t325 0 0.1f
CT326 t326 0 0.1f
CT327 t327 0 0.1f
M793 t325 nq36 vdd vdd pch w=2u l=180n
M794 t325 nw72 vdd vdd pch w=2u l=180n
CT328 t328 0 0.1f
M795 t325 nq36 t328 0 nch w=1u l=180n
M796 t328 nw72 0 0 nch w=1u l=180n
M797 t326 nq36 vdd vdd pch w=2u l=180n
M798 t326 t325 vdd vdd pch w=2u l=180n
CT329 t329 0 0.1f
M799 t326 nq36 t329 0 nch w=1u l=180n
M800 t329 t325 0 0 nch w=1u l=180n
M801 t327 nw72 vdd vdd pch w=2u l=180n
M802 t327 t325 vdd vdd pch w=2u l=180n
CT330 t330 0 0.1f
M803 t327 nw72 t330 0 nch w=1u l=180n
M804 t330 t325 0 0 nch w=1u l=180n
M805 nw73 t326 vdd vdd pch w=2u l=180n
M806 nw73 t327 vdd vdd pch w=2u l=180n
CT331 t331 0 0.1f
M807 nw73 t326 t331 0 nch w=1u l=180n
M808 t331 t327 0 0 nch w=1u l=180n
Cnw73 nw73 0 2f
CT332 t332 0 0.1f
M809 t332 nw72 vdd vdd pch w=2u l=180n
M810 t332 nq36 vdd vdd pch w=2u l=180n
CT333 t333 0 0.1f
M811 t332 nw72 t333 0 nch w=1u l=180n
M812 t333 nq36 0 0 nch w=1u l=180n
M813 nw74 t332 vdd vdd pch w=2u l=180n
M814 nw74 t332 0 0 nch w=1u l=180n
Cnw74 nw74 0 2f
CT334 t334 0 0.1f
CT335 t335 0 0.1f
CT336 t336 0 0.1f
M815 t334 nq37 vdd vdd pch w=2u l=180n
M816 t334 nw74 vdd vdd pch w=2u l=180n
CT337 t337 0 0.1f
M817 t334 nq37 t337 0 nch w=1u l=180n
M818 t337 nw74 0 0 nch w=1u l=180n
M819 t335 nq37 vdd vdd pch w=2u l=180n
M820 t335 t334 vdd vdd pch w=2u l=180n
CT338 t338 0 0.1f
M821 t335 nq37 t338 0 nch w=1u l=180n
M822 t338 t334 0 0 nch w=1u l=180n
M823 t336 nw74 vdd vdd pch w=2u l=180n
M824 t336 t334 vdd vdd pch w=2u l=180n
CT339 t339 0 0.1f
M825 t336 nw74 t339 0 nch w=1u l=180n
M826 t339 t334 0 0 nch w=1u l=180n
M827 nw75 t335 vdd vdd pch w=2u l=180n
M828 nw75 t336 vdd vdd pch w=2u l=180n
CT340 t340 0 0.1f
M829 nw75 t335 t340 0 nch w=1u l=180n
M830 t340 t336 0 0 nch w=1u l=180n
Cnw75 nw75 0 2f
CT341 t341 0 0.1f
M831 t341 nw74 vdd vdd pch w=2u l=180n
M832 t341 nq37 vdd vdd pch w=2u l=180n
CT342 t342 0 0.1f
M833 t341 nw74 t342 0 nch w=1u l=180n
M834 t342 nq37 0 0 nch w=1u l=180n
M835 nw76 t341 vdd vdd pch w=2u l=180n
M836 nw76 t341 0 0 nch w=1u l=180n
Cnw76 nw76 0 2f
CT343 t343 0 0.1f
CT344 t344 0 0.1f
CT345 t345 0 0.1f
M837 t343 nq38 vdd vdd pch w=2u l=180n
M838 t343 nw76 vdd vdd pch w=2u l=180n
CT346 t346 0 0.1f
M839 t343 nq38 t346 0 nch w=1u l=180n
M840 t346 nw76 0 0 nch w=1u l=180n
M841 t344 nq38 vdd vdd pch w=2u l=180n
M842 t344 t343 vdd vdd pch w=2u l=180n
CT347 t347 0 0.1f
M843 t344 nq38 t347 0 nch w=1u l=180n
M844 t347 t343 0 0 nch w=1u l=180n
M845 t345 nw76 vdd vdd pch w=2u l=180n
M846 t345 t343 vdd vdd pch w=2u l=180n
CT348 t348 0 0.1f
M847 t345 nw76 t348 0 nch w=1u l=180n
M848 t348 t343 0 0 nch w=1u l=180n
M849 nw77 t344 vdd vdd pch w=2u l=180n
M850 nw77 t345 vdd vdd pch w=2u l=180n
CT349 t349 0 0.1f
M851 nw77 t344 t349 0 nch w=1u l=180n
M852 t349 t345 0 0 nch w=1u l=180n
Cnw77 nw77 0 2f
CT350 t350 0 0.1f
M853 t350 nw76 vdd vdd pch w=2u l=180n
M854 t350 nq38 vdd vdd pch w=2u l=180n
CT351 t351 0 0.1f
M855 t350 nw76 t351 0 nch w=1u l=180n
M856 t351 nq38 0 0 nch w=1u l=180n
M857 nw78 t350 vdd vdd pch w=2u l=180n
M858 nw78 t350 0 0 nch w=1u l=180n
Cnw78 nw78 0 2f
CT352 t352 0 0.1f
CT353 t353 0 0.1f
CT354 t354 0 0.1f
M859 t352 nq39 vdd vdd pch w=2u l=180n
M860 t352 nw78 vdd vdd pch w=2u l=180n
CT355 t355 0 0.1f
M861 t352 nq39 t355 0 nch w=1u l=180n
M862 t355 nw78 0 0 nch w=1u l=180n
M863 t353 nq39 vdd vdd pch w=2u l=180n
M864 t353 t352 vdd vdd pch w=2u l=180n
CT356 t356 0 0.1f
M865 t353 nq39 t356 0 nch w=1u l=180n
M866 t356 t352 0 0 nch w=1u l=180n
M867 t354 nw78 vdd vdd pch w=2u l=180n
M868 t354 t352 vdd vdd pch w=2u l=180n
CT357 t357 0 0.1f
M869 t354 nw78 t357 0 nch w=1u l=180n
M870 t357 t352 0 0 nch w=1u l=180n
M871 nw79 t353 vdd vdd pch w=2u l=180n
M872 nw79 t354 vdd vdd pch w=2u l=180n
CT358 t358 0 0.1f
M873 nw79 t353 t358 0 nch w=1u l=180n
M874 t358 t354 0 0 nch w=1u l=180n
Cnw79 nw79 0 2f
CT359 t359 0 0.1f
M875 t359 nw78 vdd vdd pch w=2u l=180n
M876 t359 nq39 vdd vdd pch w=2u l=180n
CT360 t360 0 0.1f
M877 t359 nw78 t360 0 nch w=1u l=180n
M878 t360 nq39 0 0 nch w=1u l=180n
M879 nw80 t359 vdd vdd pch w=2u l=180n
M880 nw80 t359 0 0 nch w=1u l=180n
Cnw80 nw80 0 2f
CT361 t361 0 0.1f
CT362 t362 0 0.1f
CT363 t363 0 0.1f
M881 t361 nq40 vdd vdd pch w=2u l=180n
M882 t361 nw80 vdd vdd pch w=2u l=180n
CT364 t364 0 0.1f
M883 t361 nq40 t364 0 nch w=1u l=180n
M884 t364 nw80 0 0 nch w=1u l=180n
M885 t362 nq40 vdd vdd pch w=2u l=180n
M886 t362 t361 vdd vdd pch w=2u l=180n
CT365 t365 0 0.1f
M887 t362 nq40 t365 0 nch w=1u l=180n
M888 t365 t361 0 0 nch w=1u l=180n
M889 t363 nw80 vdd vdd pch w=2u l=180n
M890 t363 t361 vdd vdd pch w=2u l=180n
CT366 t366 0 0.1f
M891 t363 nw80 t366 0 nch w=1u l=180n
M892 t366 t361 0 0 nch w=1u l=180n
M893 nw81 t362 vdd vdd pch w=2u l=180n
M894 nw81 t363 vdd vdd pch w=2u l=180n
CT367 t367 0 0.1f
M895 nw81 t362 t367 0 nch w=1u l=180n
M896 t367 t363 0 0 nch w=1u l=180n
Cnw81 nw81 0 2f
CT368 t368 0 0.1f
M897 t368 nw80 vdd vdd pch w=2u l=180n
M898 t368 nq40 vdd vdd pch w=2u l=180n
CT369 t369 0 0.1f
M899 t368 nw80 t369 0 nch w=1u l=180n
M900 t369 nq40 0 0 nch w=1u l=180n
M901 nw82 t368 vdd vdd pch w=2u l=180n
M902 nw82 t368 0 0 nch w=1u l=180n
Cnw82 nw82 0 2f
CT370 t370 0 0.1f
CT371 t371 0 0.1f
CT372 t372 0 0.1f
M903 t370 nq41 vdd vdd pch w=2u l=180n
M904 t370 nw82 vdd vdd pch w=2u l=180n
CT373 t373 0 0.1f
M905 t370 nq41 t373 0 nch w=1u l=180n
M906 t373 nw82 0 0 nch w=1u l=180n
M907 t371 nq41 vdd vdd pch w=2u l=180n
M908 t371 t370 vdd vdd pch w=2u l=180n
CT374 t374 0 0.1f
M909 t371 nq41 t374 0 nch w=1u l=180n
M910 t374 t370 0 0 nch w=1u l=180n
M911 t372 nw82 vdd vdd pch w=2u l=180n
M912 t372 t370 vdd vdd pch w=2u l=180n
CT375 t375 0 0.1f
M913 t372 nw82 t375 0 nch w=1u l=180n
M914 t375 t370 0 0 nch w=1u l=180n
M915 nw83 t371 vdd vdd pch w=2u l=180n
M916 nw83 t372 vdd vdd pch w=2u l=180n
CT376 t376 0 0.1f
M917 nw83 t371 t376 0 nch w=1u l=180n
M918 t376 t372 0 0 nch w=1u l=180n
Cnw83 nw83 0 2f
CT377 t377 0 0.1f
M919 t377 nw82 vdd vdd pch w=2u l=180n
M920 t377 nq41 vdd vdd pch w=2u l=180n
CT378 t378 0 0.1f
M921 t377 nw82 t378 0 nch w=1u l=180n
M922 t378 nq41 0 0 nch w=1u l=180n
M923 nw84 t377 vdd vdd pch w=2u l=180n
M924 nw84 t377 0 0 nch w=1u l=180n
Cnw84 nw84 0 2f
CT379 t379 0 0.1f
CT380 t380 0 0.1f
CT381 t381 0 0.1f
M925 t379 nq42 vdd vdd pch w=2u l=180n
M926 t379 nw84 vdd vdd pch w=2u l=180n
CT382 t382 0 0.1f
M927 t379 nq42 t382 0 nch w=1u l=180n
M928 t382 nw84 0 0 nch w=1u l=180n
M929 t380 nq42 vdd vdd pch w=2u l=180n
M930 t380 t379 vdd vdd pch w=2u l=180n
CT383 t383 0 0.1f
M931 t380 nq42 t383 0 nch w=1u l=180n
M932 t383 t379 0 0 nch w=1u l=180n
M933 t381 nw84 vdd vdd pch w=2u l=180n
M934 t381 t379 vdd vdd pch w=2u l=180n
CT384 t384 0 0.1f
M935 t381 nw84 t384 0 nch w=1u l=180n
M936 t384 t379 0 0 nch w=1u l=180n
M937 nw85 t380 vdd vdd pch w=2u l=180n
M938 nw85 t381 vdd vdd pch w=2u l=180n
CT385 t385 0 0.1f
M939 nw85 t380 t385 0 nch w=1u l=180n
M940 t385 t381 0 0 nch w=1u l=180n
Cnw85 nw85 0 2f
CT386 t386 0 0.1f
M941 t386 nw84 vdd vdd pch w=2u l=180n
M942 t386 nq42 vdd vdd pch w=2u l=180n
CT387 t387 0 0.1f
M943 t386 nw84 t387 0 nch w=1u l=180n
M944 t387 nq42 0 0 nch w=1u l=180n
M945 nw86 t386 vdd vdd pch w=2u l=180n
M946 nw86 t386 0 0 nch w=1u l=180n
Cnw86 nw86 0 2f
CT388 t388 0 0.1f
CT389 t389 0 0.1f
CT390 t390 0 0.1f
M947 t388 nq43 vdd vdd pch w=2u l=180n
M948 t388 nw86 vdd vdd pch w=2u l=180n
CT391 t391 0 0.1f
M949 t388 nq43 t391 0 nch w=1u l=180n
M950 t391 nw86 0 0 nch w=1u l=180n
M951 t389 nq43 vdd vdd pch w=2u l=180n
M952 t389 t388 vdd vdd pch w=2u l=180n
CT392 t392 0 0.1f
M953 t389 nq43 t392 0 nch w=1u l=180n
M954 t392 t388 0 0 nch w=1u l=180n
M955 t390 nw86 vdd vdd pch w=2u l=180n
M956 t390 t388 vdd vdd pch w=2u l=180n
CT393 t393 0 0.1f
M957 t390 nw86 t393 0 nch w=1u l=180n
M958 t393 t388 0 0 nch w=1u l=180n
M959 nw87 t389 vdd vdd pch w=2u l=180n
M960 nw87 t390 vdd vdd pch w=2u l=180n
CT394 t394 0 0.1f
M961 nw87 t389 t394 0 nch w=1u l=180n
M962 t394 t390 0 0 nch w=1u l=180n
Cnw87 nw87 0 2f
CT395 t395 0 0.1f
M963 t395 nw86 vdd vdd pch w=2u l=180n
M964 t395 nq43 vdd vdd pch w=2u l=180n
CT396 t396 0 0.1f
M965 t395 nw86 t396 0 nch w=1u l=180n
M966 t396 nq43 0 0 nch w=1u l=180n
M967 nw88 t395 vdd vdd pch w=2u l=180n
M968 nw88 t395 0 0 nch w=1u l=180n
Cnw88 nw88 0 2f
CT397 t397 0 0.1f
CT398 t398 0 0.1f
CT399 t399 0 0.1f
M969 t397 nq44 vdd vdd pch w=2u l=180n
M970 t397 nw88 vdd vdd pch w=2u l=180n
CT400 t400 0 0.1f
M971 t397 nq44 t400 0 nch w=1u l=180n
M972 t400 nw88 0 0 nch w=1u l=180n
M973 t398 nq44 vdd vdd pch w=2u l=180n
M974 t398 t397 vdd vdd pch w=2u l=180n
CT401 t401 0 0.1f
M975 t398 nq44 t401 0 nch w=1u l=180n
M976 t401 t397 0 0 nch w=1u l=180n
M977 t399 nw88 vdd vdd pch w=2u l=180n
M978 t399 t397 vdd vdd pch w=2u l=180n
CT402 t402 0 0.1f
M979 t399 nw88 t402 0 nch w=1u l=180n
M980 t402 t397 0 0 nch w=1u l=180n
M981 nw89 t398 vdd vdd pch w=2u l=180n
M982 nw89 t399 vdd vdd pch w=2u l=180n
CT403 t403 0 0.1f
M983 nw89 t398 t403 0 nch w=1u l=180n
M984 t403 t399 0 0 nch w=1u l=180n
Cnw89 nw89 0 2f
CT404 t404 0 0.1f
M985 t404 nw88 vdd vdd pch w=2u l=180n
M986 t404 nq44 vdd vdd pch w=2u l=180n
CT405 t405 0 0.1f
M987 t404 nw88 t405 0 nch w=1u l=180n
M988 t405 nq44 0 0 nch w=1u l=180n
M989 nw90 t404 vdd vdd pch w=2u l=180n
M990 nw90 t404 0 0 nch w=1u l=180n
Cnw90 nw90 0 2f
CT406 t406 0 0.1f
CT407 t407 0 0.1f
CT408 t408 0 0.1f
M991 t406 nq45 vdd vdd pch w=2u l=180n
M992 t406 nw90 vdd vdd pch w=2u l=180n
CT409 t409 0 0.1f
M993 t406 nq45 t409 0 nch w=1u l=180n
M994 t409 nw90 0 0 nch w=1u l=180n
M995 t407 nq45 vdd vdd pch w=2u l=180n
M996 t407 t406 vdd vdd pch w=2u l=180n
CT410 t410 0 0.1f
M997 t407 nq45 t410 0 nch w=1u l=180n
M998 t410 t406 0 0 nch w=1u l=180n
M999 t408 nw90 vdd vdd pch w=2u l=180n
M1000 t408 t406 vdd vdd pch w=2u l=180n
CT411 t411 0 0.1f
M1001 t408 nw90 t411 0 nch w=1u l=180n
M1002 t411 t406 0 0 nch w=1u l=180n
M1003 nw91 t407 vdd vdd pch w=2u l=180n
M1004 nw91 t408 vdd vdd pch w=2u l=180n
CT412 t412 0 0.1f
M1005 nw91 t407 t412 0 nch w=1u l=180n
M1006 t412 t408 0 0 nch w=1u l=180n
Cnw91 nw91 0 2f
CT413 t413 0 0.1f
M1007 t413 nw90 vdd vdd pch w=2u l=180n
M1008 t413 nq45 vdd vdd pch w=2u l=180n
CT414 t414 0 0.1f
M1009 t413 nw90 t414 0 nch w=1u l=180n
M1010 t414 nq45 0 0 nch w=1u l=180n
M1011 nw92 t413 vdd vdd pch w=2u l=180n
M1012 nw92 t413 0 0 nch w=1u l=180n
Cnw92 nw92 0 2f
CT415 t415 0 0.1f
CT416 t416 0 0.1f
CT417 t417 0 0.1f
M1013 t415 nq46 vdd vdd pch w=2u l=180n
M1014 t415 nw92 vdd vdd pch w=2u l=180n
CT418 t418 0 0.1f
M1015 t415 nq46 t418 0 nch w=1u l=180n
M1016 t418 nw92 0 0 nch w=1u l=180n
M1017 t416 nq46 vdd vdd pch w=2u l=180n
M1018 t416 t415 vdd vdd pch w=2u l=180n
CT419 t419 0 0.1f
M1019 t416 nq46 t419 0 nch w=1u l=180n
M1020 t419 t415 0 0 nch w=1u l=180n
M1021 t417 nw92 vdd vdd pch w=2u l=180n
M1022 t417 t415 vdd vdd pch w=2u l=180n
CT420 t420 0 0.1f
M1023 t417 nw92 t420 0 nch w=1u l=180n
M1024 t420 t415 0 0 nch w=1u l=180n
M1025 nw93 t416 vdd vdd pch w=2u l=180n
M1026 nw93 t417 vdd vdd pch w=2u l=180n
CT421 t421 0 0.1f
M1027 nw93 t416 t421 0 nch w=1u l=180n
M1028 t421 t417 0 0 nch w=1u l=180n
Cnw93 nw93 0 2f
CT422 t422 0 0.1f
M1029 t422 nw92 vdd vdd pch w=2u l=180n
M1030 t422 nq46 vdd vdd pch w=2u l=180n
CT423 t423 0 0.1f
M1031 t422 nw92 t423 0 nch w=1u l=180n
M1032 t423 nq46 0 0 nch w=1u l=180n
M1033 nw94 t422 vdd vdd pch w=2u l=180n
M1034 nw94 t422 0 0 nch w=1u l=180n
Cnw94 nw94 0 2f
CT424 t424 0 0.1f
CT425 t425 0 0.1f
CT426 t426 0 0.1f
M1035 t424 nq47 vdd vdd pch w=2u l=180n
M1036 t424 nw94 vdd vdd pch w=2u l=180n
CT427 t427 0 0.1f
M1037 t424 nq47 t427 0 nch w=1u l=180n
M1038 t427 nw94 0 0 nch w=1u l=180n
M1039 t425 nq47 vdd vdd pch w=2u l=180n
M1040 t425 t424 vdd vdd pch w=2u l=180n
CT428 t428 0 0.1f
M1041 t425 nq47 t428 0 nch w=1u l=180n
M1042 t428 t424 0 0 nch w=1u l=180n
M1043 t426 nw94 vdd vdd pch w=2u l=180n
M1044 t426 t424 vdd vdd pch w=2u l=180n
CT429 t429 0 0.1f
M1045 t426 nw94 t429 0 nch w=1u l=180n
M1046 t429 t424 0 0 nch w=1u l=180n
M1047 nw95 t425 vdd vdd pch w=2u l=180n
M1048 nw95 t426 vdd vdd pch w=2u l=180n
CT430 t430 0 0.1f
M1049 nw95 t425 t430 0 nch w=1u l=180n
M1050 t430 t426 0 0 nch w=1u l=180n
Cnw95 nw95 0 2f
CT431 t431 0 0.1f
M1051 t431 nw94 vdd vdd pch w=2u l=180n
M1052 t431 nq47 vdd vdd pch w=2u l=180n
CT432 t432 0 0.1f
M1053 t431 nw94 t432 0 nch w=1u l=180n
M1054 t432 nq47 0 0 nch w=1u l=180n
M1055 nw96 t431 vdd vdd pch w=2u l=180n
M1056 nw96 t431 0 0 nch w=1u l=180n
Cnw96 nw96 0 2f
CT433 t433 0 0.1f
CT434 t434 0 0.1f
CT435 t435 0 0.1f
M1057 t433 nq48 vdd vdd pch w=2u l=180n
M1058 t433 nw96 vdd vdd pch w=2u l=180n
CT436 t436 0 0.1f
M1059 t433 nq48 t436 0 nch w=1u l=180n
M1060 t436 nw96 0 0 nch w=1u l=180n
M1061 t434 nq48 vdd vdd pch w=2u l=180n
M1062 t434 t433 vdd vdd pch w=2u l=180n
CT437 t437 0 0.1f
M1063 t434 nq48 t437 0 nch w=1u l=180n
M1064 t437 t433 0 0 nch w=1u l=180n
M1065 t435 nw96 vdd vdd pch w=2u l=180n
M1066 t435 t433 vdd vdd pch w=2u l=180n
CT438 t438 0 0.1f
M1067 t435 nw96 t438 0 nch w=1u l=180n
M1068 t438 t433 0 0 nch w=1u l=180n
M1069 nw97 t434 vdd vdd pch w=2u l=180n
M1070 nw97 t435 vdd vdd pch w=2u l=180n
CT439 t439 0 0.1f
M1071 nw97 t434 t439 0 nch w=1u l=180n
M1072 t439 t435 0 0 nch w=1u l=180n
Cnw97 nw97 0 2f
CT440 t440 0 0.1f
M1073 t440 nw96 vdd vdd pch w=2u l=180n
M1074 t440 nq48 vdd vdd pch w=2u l=180n
CT441 t441 0 0.1f
M1075 t440 nw96 t441 0 nch w=1u l=180n
M1076 t441 nq48 0 0 nch w=1u l=180n
M1077 nw98 t440 vdd vdd pch w=2u l=180n
M1078 nw98 t440 0 0 nch w=1u l=180n
Cnw98 nw98 0 2f
CT442 t442 0 0.1f
CT443 t443 0 0.1f
CT444 t444 0 0.1f
M1079 t442 nq49 vdd vdd pch w=2u l=180n
M1080 t442 nw98 vdd vdd pch w=2u l=180n
CT445 t445 0 0.1f
M1081 t442 nq49 t445 0 nch w=1u l=180n
M1082 t445 nw98 0 0 nch w=1u l=180n
M1083 t443 nq49 vdd vdd pch w=2u l=180n
M1084 t443 t442 vdd vdd pch w=2u l=180n
CT446 t446 0 0.1f
M1085 t443 nq49 t446 0 nch w=1u l=180n
M1086 t446 t442 0 0 nch w=1u l=180n
M1087 t444 nw98 vdd vdd pch w=2u l=180n
M1088 t444 t442 vdd vdd pch w=2u l=180n
CT447 t447 0 0.1f
M1089 t444 nw98 t447 0 nch w=1u l=180n
M1090 t447 t442 0 0 nch w=1u l=180n
M1091 nw99 t443 vdd vdd pch w=2u l=180n
M1092 nw99 t444 vdd vdd pch w=2u l=180n
CT448 t448 0 0.1f
M1093 nw99 t443 t448 0 nch w=1u l=180n
M1094 t448 t444 0 0 nch w=1u l=180n
Cnw99 nw99 0 2f
CT449 t449 0 0.1f
M1095 t449 nw98 vdd vdd pch w=2u l=180n
M1096 t449 nq49 vdd vdd pch w=2u l=180n
CT450 t450 0 0.1f
M1097 t449 nw98 t450 0 nch w=1u l=180n
M1098 t450 nq49 0 0 nch w=1u l=180n
M1099 nw100 t449 vdd vdd pch w=2u l=180n
M1100 nw100 t449 0 0 nch w=1u l=180n
Cnw100 nw100 0 2f
CT451 t451 0 0.1f
CT452 t452 0 0.1f
CT453 t453 0 0.1f
M1101 t451 nq50 vdd vdd pch w=2u l=180n
M1102 t451 nw100 vdd vdd pch w=2u l=180n
CT454 t454 0 0.1f
M1103 t451 nq50 t454 0 nch w=1u l=180n
M1104 t454 nw100 0 0 nch w=1u l=180n
M1105 t452 nq50 vdd vdd pch w=2u l=180n
M1106 t452 t451 vdd vdd pch w=2u l=180n
CT455 t455 0 0.1f
M1107 t452 nq50 t455 0 nch w=1u l=180n
M1108 t455 t451 0 0 nch w=1u l=180n
M1109 t453 nw100 vdd vdd pch w=2u l=180n
M1110 t453 t451 vdd vdd pch w=2u l=180n
CT456 t456 0 0.1f
M1111 t453 nw100 t456 0 nch w=1u l=180n
M1112 t456 t451 0 0 nch w=1u l=180n
M1113 nw101 t452 vdd vdd pch w=2u l=180n
M1114 nw101 t453 vdd vdd pch w=2u l=180n
CT457 t457 0 0.1f
M1115 nw101 t452 t457 0 nch w=1u l=180n
M1116 t457 t453 0 0 nch w=1u l=180n
Cnw101 nw101 0 2f
CT458 t458 0 0.1f
M1117 t458 nw100 vdd vdd pch w=2u l=180n
M1118 t458 nq50 vdd vdd pch w=2u l=180n
CT459 t459 0 0.1f
M1119 t458 nw100 t459 0 nch w=1u l=180n
M1120 t459 nq50 0 0 nch w=1u l=180n
M1121 nw102 t458 vdd vdd pch w=2u l=180n
M1122 nw102 t458 0 0 nch w=1u l=180n
Cnw102 nw102 0 2f
CT460 t460 0 0.1f
CT461 t461 0 0.1f
CT462 t462 0 0.1f
M1123 t460 nq51 vdd vdd pch w=2u l=180n
M1124 t460 nw102 vdd vdd pch w=2u l=180n
CT463 t463 0 0.1f
M1125 t460 nq51 t463 0 nch w=1u l=180n
M1126 t463 nw102 0 0 nch w=1u l=180n
M1127 t461 nq51 vdd vdd pch w=2u l=180n
M1128 t461 t460 vdd vdd pch w=2u l=180n
CT464 t464 0 0.1f
M1129 t461 nq51 t464 0 nch w=1u l=180n
M1130 t464 t460 0 0 nch w=1u l=180n
M1131 t462 nw102 vdd vdd pch w=2u l=180n
M1132 t462 t460 vdd vdd pch w=2u l=180n
CT465 t465 0 0.1f
M1133 t462 nw102 t465 0 nch w=1u l=180n
M1134 t465 t460 0 0 nch w=1u l=180n
M1135 nw103 t461 vdd vdd pch w=2u l=180n
M1136 nw103 t462 vdd vdd pch w=2u l=180n
CT466 t466 0 0.1f
M1137 nw103 t461 t466 0 nch w=1u l=180n
M1138 t466 t462 0 0 nch w=1u l=180n
Cnw103 nw103 0 2f
CT467 t467 0 0.1f
M1139 t467 nw102 vdd vdd pch w=2u l=180n
M1140 t467 nq51 vdd vdd pch w=2u l=180n
CT468 t468 0 0.1f
M1141 t467 nw102 t468 0 nch w=1u l=180n
M1142 t468 nq51 0 0 nch w=1u l=180n
M1143 nw104 t467 vdd vdd pch w=2u l=180n
M1144 nw104 t467 0 0 nch w=1u l=180n
Cnw104 nw104 0 2f
CT469 t469 0 0.1f
CT470 t470 0 0.1f
CT471 t471 0 0.1f
M1145 t469 nq52 vdd vdd pch w=2u l=180n
M1146 t469 nw104 vdd vdd pch w=2u l=180n
CT472 t472 0 0.1f
M1147 t469 nq52 t472 0 nch w=1u l=180n
M1148 t472 nw104 0 0 nch w=1u l=180n
M1149 t470 nq52 vdd vdd pch w=2u l=180n
M1150 t470 t469 vdd vdd pch w=2u l=180n
CT473 t473 0 0.1f
M1151 t470 nq52 t473 0 nch w=1u l=180n
M1152 t473 t469 0 0 nch w=1u l=180n
M1153 t471 nw104 vdd vdd pch w=2u l=180n
M1154 t471 t469 vdd vdd pch w=2u l=180n
CT474 t474 0 0.1f
M1155 t471 nw104 t474 0 nch w=1u l=180n
M1156 t474 t469 0 0 nch w=1u l=180n
M1157 nw105 t470 vdd vdd pch w=2u l=180n
M1158 nw105 t471 vdd vdd pch w=2u l=180n
CT475 t475 0 0.1f
M1159 nw105 t470 t475 0 nch w=1u l=180n
M1160 t475 t471 0 0 nch w=1u l=180n
Cnw105 nw105 0 2f
CT476 t476 0 0.1f
M1161 t476 nw104 vdd vdd pch w=2u l=180n
M1162 t476 nq52 vdd vdd pch w=2u l=180n
CT477 t477 0 0.1f
M1163 t476 nw104 t477 0 nch w=1u l=180n
M1164 t477 nq52 0 0 nch w=1u l=180n
M1165 nw106 t476 vdd vdd pch w=2u l=180n
M1166 nw106 t476 0 0 nch w=1u l=180n
Cnw106 nw106 0 2f
CT478 t478 0 0.1f
CT479 t479 0 0.1f
CT480 t480 0 0.1f
M1167 t478 nq53 vdd vdd pch w=2u l=180n
M1168 t478 nw106 vdd vdd pch w=2u l=180n
CT481 t481 0 0.1f
M1169 t478 nq53 t481 0 nch w=1u l=180n
M1170 t481 nw106 0 0 nch w=1u l=180n
M1171 t479 nq53 vdd vdd pch w=2u l=180n
M1172 t479 t478 vdd vdd pch w=2u l=180n
CT482 t482 0 0.1f
M1173 t479 nq53 t482 0 nch w=1u l=180n
M1174 t482 t478 0 0 nch w=1u l=180n
M1175 t480 nw106 vdd vdd pch w=2u l=180n
M1176 t480 t478 vdd vdd pch w=2u l=180n
CT483 t483 0 0.1f
M1177 t480 nw106 t483 0 nch w=1u l=180n
M1178 t483 t478 0 0 nch w=1u l=180n
M1179 nw107 t479 vdd vdd pch w=2u l=180n
M1180 nw107 t480 vdd vdd pch w=2u l=180n
CT484 t484 0 0.1f
M1181 nw107 t479 t484 0 nch w=1u l=180n
M1182 t484 t480 0 0 nch w=1u l=180n
Cnw107 nw107 0 2f
CT485 t485 0 0.1f
M1183 t485 nw106 vdd vdd pch w=2u l=180n
M1184 t485 nq53 vdd vdd pch w=2u l=180n
CT486 t486 0 0.1f
M1185 t485 nw106 t486 0 nch w=1u l=180n
M1186 t486 nq53 0 0 nch w=1u l=180n
M1187 nw108 t485 vdd vdd pch w=2u l=180n
M1188 nw108 t485 0 0 nch w=1u l=180n
Cnw108 nw108 0 2f
CT487 t487 0 0.1f
CT488 t488 0 0.1f
CT489 t489 0 0.1f
M1189 t487 nq54 vdd vdd pch w=2u l=180n
M1190 t487 nw108 vdd vdd pch w=2u l=180n
CT490 t490 0 0.1f
M1191 t487 nq54 t490 0 nch w=1u l=180n
M1192 t490 nw108 0 0 nch w=1u l=180n
M1193 t488 nq54 vdd vdd pch w=2u l=180n
M1194 t488 t487 vdd vdd pch w=2u l=180n
CT491 t491 0 0.1f
M1195 t488 nq54 t491 0 nch w=1u l=180n
M1196 t491 t487 0 0 nch w=1u l=180n
M1197 t489 nw108 vdd vdd pch w=2u l=180n
M1198 t489 t487 vdd vdd pch w=2u l=180n
CT492 t492 0 0.1f
M1199 t489 nw108 t492 0 nch w=1u l=180n
M1200 t492 t487 0 0 nch w=1u l=180n
M1201 nw109 t488 vdd vdd pch w=2u l=180n
M1202 nw109 t489 vdd vdd pch w=2u l=180n
CT493 t493 0 0.1f
M1203 nw109 t488 t493 0 nch w=1u l=180n
M1204 t493 t489 0 0 nch w=1u l=180n
Cnw109 nw109 0 2f
CT494 t494 0 0.1f
M1205 t494 nw108 vdd vdd pch w=2u l=180n
M1206 t494 nq54 vdd vdd pch w=2u l=180n
CT495 t495 0 0.1f
M1207 t494 nw108 t495 0 nch w=1u l=180n
M1208 t495 nq54 0 0 nch w=1u l=180n
M1209 nw110 t494 vdd vdd pch w=2u l=180n
M1210 nw110 t494 0 0 nch w=1u l=180n
Cnw110 nw110 0 2f
CT496 t496 0 0.1f
CT497 t497 0 0.1f
CT498 t498 0 0.1f
M1211 t496 nq55 vdd vdd pch w=2u l=180n
M1212 t496 nw110 vdd vdd pch w=2u l=180n
CT499 t499 0 0.1f
M1213 t496 nq55 t499 0 nch w=1u l=180n
M1214 t499 nw110 0 0 nch w=1u l=180n
M1215 t497 nq55 vdd vdd pch w=2u l=180n
M1216 t497 t496 vdd vdd pch w=2u l=180n
CT500 t500 0 0.1f
M1217 t497 nq55 t500 0 nch w=1u l=180n
M1218 t500 t496 0 0 nch w=1u l=180n
M1219 t498 nw110 vdd vdd pch w=2u l=180n
M1220 t498 t496 vdd vdd pch w=2u l=180n
CT501 t501 0 0.1f
M1221 t498 nw110 t501 0 nch w=1u l=180n
M1222 t501 t496 0 0 nch w=1u l=180n
M1223 nw111 t497 vdd vdd pch w=2u l=180n
M1224 nw111 t498 vdd vdd pch w=2u l=180n
CT502 t502 0 0.1f
M1225 nw111 t497 t502 0 nch w=1u l=180n
M1226 t502 t498 0 0 nch w=1u l=180n
Cnw111 nw111 0 2f
CT503 t503 0 0.1f
M1227 t503 nw110 vdd vdd pch w=2u l=180n
M1228 t503 nq55 vdd vdd pch w=2u l=180n
CT504 t504 0 0.1f
M1229 t503 nw110 t504 0 nch w=1u l=180n
M1230 t504 nq55 0 0 nch w=1u l=180n
M1231 nw112 t503 vdd vdd pch w=2u l=180n
M1232 nw112 t503 0 0 nch w=1u l=180n
Cnw112 nw112 0 2f
CT505 t505 0 0.1f
CT506 t506 0 0.1f
CT507 t507 0 0.1f
M1233 t505 nq56 vdd vdd pch w=2u l=180n
M1234 t505 nw112 vdd vdd pch w=2u l=180n
CT508 t508 0 0.1f
M1235 t505 nq56 t508 0 nch w=1u l=180n
M1236 t508 nw112 0 0 nch w=1u l=180n
M1237 t506 nq56 vdd vdd pch w=2u l=180n
M1238 t506 t505 vdd vdd pch w=2u l=180n
CT509 t509 0 0.1f
M1239 t506 nq56 t509 0 nch w=1u l=180n
M1240 t509 t505 0 0 nch w=1u l=180n
M1241 t507 nw112 vdd vdd pch w=2u l=180n
M1242 t507 t505 vdd vdd pch w=2u l=180n
CT510 t510 0 0.1f
M1243 t507 nw112 t510 0 nch w=1u l=180n
M1244 t510 t505 0 0 nch w=1u l=180n
M1245 nw113 t506 vdd vdd pch w=2u l=180n
M1246 nw113 t507 vdd vdd pch w=2u l=180n
CT511 t511 0 0.1f
M1247 nw113 t506 t511 0 nch w=1u l=180n
M1248 t511 t507 0 0 nch w=1u l=180n
Cnw113 nw113 0 2f
CT512 t512 0 0.1f
M1249 t512 nw112 vdd vdd pch w=2u l=180n
M1250 t512 nq56 vdd vdd pch w=2u l=180n
CT513 t513 0 0.1f
M1251 t512 nw112 t513 0 nch w=1u l=180n
M1252 t513 nq56 0 0 nch w=1u l=180n
M1253 nw114 t512 vdd vdd pch w=2u l=180n
M1254 nw114 t512 0 0 nch w=1u l=180n
Cnw114 nw114 0 2f
CT514 t514 0 0.1f
CT515 t515 0 0.1f
CT516 t516 0 0.1f
M1255 t514 nq57 vdd vdd pch w=2u l=180n
M1256 t514 nw114 vdd vdd pch w=2u l=180n
CT517 t517 0 0.1f
M1257 t514 nq57 t517 0 nch w=1u l=180n
M1258 t517 nw114 0 0 nch w=1u l=180n
M1259 t515 nq57 vdd vdd pch w=2u l=180n
M1260 t515 t514 vdd vdd pch w=2u l=180n
CT518 t518 0 0.1f
M1261 t515 nq57 t518 0 nch w=1u l=180n
M1262 t518 t514 0 0 nch w=1u l=180n
M1263 t516 nw114 vdd vdd pch w=2u l=180n
M1264 t516 t514 vdd vdd pch w=2u l=180n
CT519 t519 0 0.1f
M1265 t516 nw114 t519 0 nch w=1u l=180n
M1266 t519 t514 0 0 nch w=1u l=180n
M1267 nw115 t515 vdd vdd pch w=2u l=180n
M1268 nw115 t516 vdd vdd pch w=2u l=180n
CT520 t520 0 0.1f
M1269 nw115 t515 t520 0 nch w=1u l=180n
M1270 t520 t516 0 0 nch w=1u l=180n
Cnw115 nw115 0 2f
CT521 t521 0 0.1f
M1271 t521 nw114 vdd vdd pch w=2u l=180n
M1272 t521 nq57 vdd vdd pch w=2u l=180n
CT522 t522 0 0.1f
M1273 t521 nw114 t522 0 nch w=1u l=180n
M1274 t522 nq57 0 0 nch w=1u l=180n
M1275 nw116 t521 vdd vdd pch w=2u l=180n
M1276 nw116 t521 0 0 nch w=1u l=180n
Cnw116 nw116 0 2f
CT523 t523 0 0.1f
CT524 t524 0 0.1f
CT525 t525 0 0.1f
M1277 t523 nq58 vdd vdd pch w=2u l=180n
M1278 t523 nw116 vdd vdd pch w=2u l=180n
CT526 t526 0 0.1f
M1279 t523 nq58 t526 0 nch w=1u l=180n
M1280 t526 nw116 0 0 nch w=1u l=180n
M1281 t524 nq58 vdd vdd pch w=2u l=180n
M1282 t524 t523 vdd vdd pch w=2u l=180n
CT527 t527 0 0.1f
M1283 t524 nq58 t527 0 nch w=1u l=180n
M1284 t527 t523 0 0 nch w=1u l=180n
M1285 t525 nw116 vdd vdd pch w=2u l=180n
M1286 t525 t523 vdd vdd pch w=2u l=180n
CT528 t528 0 0.1f
M1287 t525 nw116 t528 0 nch w=1u l=180n
M1288 t528 t523 0 0 nch w=1u l=180n
M1289 nw117 t524 vdd vdd pch w=2u l=180n
M1290 nw117 t525 vdd vdd pch w=2u l=180n
CT529 t529 0 0.1f
M1291 nw117 t524 t529 0 nch w=1u l=180n
M1292 t529 t525 0 0 nch w=1u l=180n
Cnw117 nw117 0 2f
CT530 t530 0 0.1f
M1293 t530 nw116 vdd vdd pch w=2u l=180n
M1294 t530 nq58 vdd vdd pch w=2u l=180n
CT531 t531 0 0.1f
M1295 t530 nw116 t531 0 nch w=1u l=180n
M1296 t531 nq58 0 0 nch w=1u l=180n
M1297 nw118 t530 vdd vdd pch w=2u l=180n
M1298 nw118 t530 0 0 nch w=1u l=180n
Cnw118 nw118 0 2f
CT532 t532 0 0.1f
CT533 t533 0 0.1f
CT534 t534 0 0.1f
M1299 t532 nq59 vdd vdd pch w=2u l=180n
M1300 t532 nw118 vdd vdd pch w=2u l=180n
CT535 t535 0 0.1f
M1301 t532 nq59 t535 0 nch w=1u l=180n
M1302 t535 nw118 0 0 nch w=1u l=180n
M1303 t533 nq59 vdd vdd pch w=2u l=180n
M1304 t533 t532 vdd vdd pch w=2u l=180n
CT536 t536 0 0.1f
M1305 t533 nq59 t536 0 nch w=1u l=180n
M1306 t536 t532 0 0 nch w=1u l=180n
M1307 t534 nw118 vdd vdd pch w=2u l=180n
M1308 t534 t532 vdd vdd pch w=2u l=180n
CT537 t537 0 0.1f
M1309 t534 nw118 t537 0 nch w=1u l=180n
M1310 t537 t532 0 0 nch w=1u l=180n
M1311 nw119 t533 vdd vdd pch w=2u l=180n
M1312 nw119 t534 vdd vdd pch w=2u l=180n
CT538 t538 0 0.1f
M1313 nw119 t533 t538 0 nch w=1u l=180n
M1314 t538 t534 0 0 nch w=1u l=180n
Cnw119 nw119 0 2f
CT539 t539 0 0.1f
M1315 t539 nw118 vdd vdd pch w=2u l=180n
M1316 t539 nq59 vdd vdd pch w=2u l=180n
CT540 t540 0 0.1f
M1317 t539 nw118 t540 0 nch w=1u l=180n
M1318 t540 nq59 0 0 nch w=1u l=180n
M1319 nw120 t539 vdd vdd pch w=2u l=180n
M1320 nw120 t539 0 0 nch w=1u l=180n
Cnw120 nw120 0 2f
CT541 t541 0 0.1f
CT542 t542 0 0.1f
CT543 t543 0 0.1f
M1321 t541 nq60 vdd vdd pch w=2u l=180n
M1322 t541 nw120 vdd vdd pch w=2u l=180n
CT544 t544 0 0.1f
M1323 t541 nq60 t544 0 nch w=1u l=180n
M1324 t544 nw120 0 0 nch w=1u l=180n
M1325 t542 nq60 vdd vdd pch w=2u l=180n
M1326 t542 t541 vdd vdd pch w=2u l=180n
CT545 t545 0 0.1f
M1327 t542 nq60 t545 0 nch w=1u l=180n
M1328 t545 t541 0 0 nch w=1u l=180n
M1329 t543 nw120 vdd vdd pch w=2u l=180n
M1330 t543 t541 vdd vdd pch w=2u l=180n
CT546 t546 0 0.1f
M1331 t543 nw120 t546 0 nch w=1u l=180n
M1332 t546 t541 0 0 nch w=1u l=180n
M1333 nw121 t542 vdd vdd pch w=2u l=180n
M1334 nw121 t543 vdd vdd pch w=2u l=180n
CT547 t547 0 0.1f
M1335 nw121 t542 t547 0 nch w=1u l=180n
M1336 t547 t543 0 0 nch w=1u l=180n
Cnw121 nw121 0 2f
CT548 t548 0 0.1f
M1337 t548 nw120 vdd vdd pch w=2u l=180n
M1338 t548 nq60 vdd vdd pch w=2u l=180n
CT549 t549 0 0.1f
M1339 t548 nw120 t549 0 nch w=1u l=180n
M1340 t549 nq60 0 0 nch w=1u l=180n
M1341 nw122 t548 vdd vdd pch w=2u l=180n
M1342 nw122 t548 0 0 nch w=1u l=180n
Cnw122 nw122 0 2f
CT550 t550 0 0.1f
CT551 t551 0 0.1f
CT552 t552 0 0.1f
M1343 t550 nq61 vdd vdd pch w=2u l=180n
M1344 t550 nw122 vdd vdd pch w=2u l=180n
CT553 t553 0 0.1f
M1345 t550 nq61 t553 0 nch w=1u l=180n
M1346 t553 nw122 0 0 nch w=1u l=180n
M1347 t551 nq61 vdd vdd pch w=2u l=180n
M1348 t551 t550 vdd vdd pch w=2u l=180n
CT554 t554 0 0.1f
M1349 t551 nq61 t554 0 nch w=1u l=180n
M1350 t554 t550 0 0 nch w=1u l=180n
M1351 t552 nw122 vdd vdd pch w=2u l=180n
M1352 t552 t550 vdd vdd pch w=2u l=180n
CT555 t555 0 0.1f
M1353 t552 nw122 t555 0 nch w=1u l=180n
M1354 t555 t550 0 0 nch w=1u l=180n
M1355 nw123 t551 vdd vdd pch w=2u l=180n
M1356 nw123 t552 vdd vdd pch w=2u l=180n
CT556 t556 0 0.1f
M1357 nw123 t551 t556 0 nch w=1u l=180n
M1358 t556 t552 0 0 nch w=1u l=180n
Cnw123 nw123 0 2f
CT557 t557 0 0.1f
M1359 t557 nw122 vdd vdd pch w=2u l=180n
M1360 t557 nq61 vdd vdd pch w=2u l=180n
CT558 t558 0 0.1f
M1361 t557 nw122 t558 0 nch w=1u l=180n
M1362 t558 nq61 0 0 nch w=1u l=180n
M1363 nw124 t557 vdd vdd pch w=2u l=180n
M1364 nw124 t557 0 0 nch w=1u l=180n
Cnw124 nw124 0 2f
CT559 t559 0 0.1f
CT560 t560 0 0.1f
CT561 t561 0 0.1f
M1365 t559 nq62 vdd vdd pch w=2u l=180n
M1366 t559 nw124 vdd vdd pch w=2u l=180n
CT562 t562 0 0.1f
M1367 t559 nq62 t562 0 nch w=1u l=180n
M1368 t562 nw124 0 0 nch w=1u l=180n
M1369 t560 nq62 vdd vdd pch w=2u l=180n
M1370 t560 t559 vdd vdd pch w=2u l=180n
CT563 t563 0 0.1f
M1371 t560 nq62 t563 0 nch w=1u l=180n
M1372 t563 t559 0 0 nch w=1u l=180n
M1373 t561 nw124 vdd vdd pch w=2u l=180n
M1374 t561 t559 vdd vdd pch w=2u l=180n
CT564 t564 0 0.1f
M1375 t561 nw124 t564 0 nch w=1u l=180n
M1376 t564 t559 0 0 nch w=1u l=180n
M1377 nw125 t560 vdd vdd pch w=2u l=180n
M1378 nw125 t561 vdd vdd pch w=2u l=180n
CT565 t565 0 0.1f
M1379 nw125 t560 t565 0 nch w=1u l=180n
M1380 t565 t561 0 0 nch w=1u l=180n
Cnw125 nw125 0 2f
CT566 t566 0 0.1f
M1381 t566 nw124 vdd vdd pch w=2u l=180n
M1382 t566 nq62 vdd vdd pch w=2u l=180n
CT567 t567 0 0.1f
M1383 t566 nw124 t567 0 nch w=1u l=180n
M1384 t567 nq62 0 0 nch w=1u l=180n
M1385 nw126 t566 vdd vdd pch w=2u l=180n
M1386 nw126 t566 0 0 nch w=1u l=180n
Cnw126 nw126 0 2f
CT568 t568 0 0.1f
CT569 t569 0 0.1f
CT570 t570 0 0.1f
M1387 t568 nq63 vdd vdd pch w=2u l=180n
M1388 t568 nw126 vdd vdd pch w=2u l=180n
CT571 t571 0 0.1f
M1389 t568 nq63 t571 0 nch w=1u l=180n
M1390 t571 nw126 0 0 nch w=1u l=180n
M1391 t569 nq63 vdd vdd pch w=2u l=180n
M1392 t569 t568 vdd vdd pch w=2u l=180n
CT572 t572 0 0.1f
M1393 t569 nq63 t572 0 nch w=1u l=180n
M1394 t572 t568 0 0 nch w=1u l=180n
M1395 t570 nw126 vdd vdd pch w=2u l=180n
M1396 t570 t568 vdd vdd pch w=2u l=180n
CT573 t573 0 0.1f
M1397 t570 nw126 t573 0 nch w=1u l=180n
M1398 t573 t568 0 0 nch w=1u l=180n
M1399 nw127 t569 vdd vdd pch w=2u l=180n
M1400 nw127 t570 vdd vdd pch w=2u l=180n
CT574 t574 0 0.1f
M1401 nw127 t569 t574 0 nch w=1u l=180n
M1402 t574 t570 0 0 nch w=1u l=180n
Cnw127 nw127 0 2f
CT575 t575 0 0.1f
M1403 t575 nw126 vdd vdd pch w=2u l=180n
M1404 t575 nq63 vdd vdd pch w=2u l=180n
CT576 t576 0 0.1f
M1405 t575 nw126 t576 0 nch w=1u l=180n
M1406 t576 nq63 0 0 nch w=1u l=180n
M1407 nw128 t575 vdd vdd pch w=2u l=180n
M1408 nw128 t575 0 0 nch w=1u l=180n
Cnw128 nw128 0 2f
CT577 t577 0 0.1f
CT578 t578 0 0.1f
CT579 t579 0 0.1f
M1409 t577 nq64 vdd vdd pch w=2u l=180n
M1410 t577 nw128 vdd vdd pch w=2u l=180n
CT580 t580 0 0.1f
M1411 t577 nq64 t580 0 nch w=1u l=180n
M1412 t580 nw128 0 0 nch w=1u l=180n
M1413 t578 nq64 vdd vdd pch w=2u l=180n
M1414 t578 t577 vdd vdd pch w=2u l=180n
CT581 t581 0 0.1f
M1415 t578 nq64 t581 0 nch w=1u l=180n
M1416 t581 t577 0 0 nch w=1u l=180n
M1417 t579 nw128 vdd vdd pch w=2u l=180n
M1418 t579 t577 vdd vdd pch w=2u l=180n
CT582 t582 0 0.1f
M1419 t579 nw128 t582 0 nch w=1u l=180n
M1420 t582 t577 0 0 nch w=1u l=180n
M1421 nw129 t578 vdd vdd pch w=2u l=180n
M1422 nw129 t579 vdd vdd pch w=2u l=180n
CT583 t583 0 0.1f
M1423 nw129 t578 t583 0 nch w=1u l=180n
M1424 t583 t579 0 0 nch w=1u l=180n
Cnw129 nw129 0 2f
CT584 t584 0 0.1f
M1425 t584 nw128 vdd vdd pch w=2u l=180n
M1426 t584 nq64 vdd vdd pch w=2u l=180n
CT585 t585 0 0.1f
M1427 t584 nw128 t585 0 nch w=1u l=180n
M1428 t585 nq64 0 0 nch w=1u l=180n
M1429 nw130 t584 vdd vdd pch w=2u l=180n
M1430 nw130 t584 0 0 nch w=1u l=180n
Cnw130 nw130 0 2f
CT586 t586 0 0.1f
CT587 t587 0 0.1f
CT588 t588 0 0.1f
M1431 t586 nq65 vdd vdd pch w=2u l=180n
M1432 t586 nw130 vdd vdd pch w=2u l=180n
CT589 t589 0 0.1f
M1433 t586 nq65 t589 0 nch w=1u l=180n
M1434 t589 nw130 0 0 nch w=1u l=180n
M1435 t587 nq65 vdd vdd pch w=2u l=180n
M1436 t587 t586 vdd vdd pch w=2u l=180n
CT590 t590 0 0.1f
M1437 t587 nq65 t590 0 nch w=1u l=180n
M1438 t590 t586 0 0 nch w=1u l=180n
M1439 t588 nw130 vdd vdd pch w=2u l=180n
M1440 t588 t586 vdd vdd pch w=2u l=180n
CT591 t591 0 0.1f
M1441 t588 nw130 t591 0 nch w=1u l=180n
M1442 t591 t586 0 0 nch w=1u l=180n
M1443 nw131 t587 vdd vdd pch w=2u l=180n
M1444 nw131 t588 vdd vdd pch w=2u l=180n
CT592 t592 0 0.1f
M1445 nw131 t587 t592 0 nch w=1u l=180n
M1446 t592 t588 0 0 nch w=1u l=180n
Cnw131 nw131 0 2f
CT593 t593 0 0.1f
M1447 t593 nw130 vdd vdd pch w=2u l=180n
M1448 t593 nq65 vdd vdd pch w=2u l=180n
CT594 t594 0 0.1f
M1449 t593 nw130 t594 0 nch w=1u l=180n
M1450 t594 nq65 0 0 nch w=1u l=180n
M1451 nw132 t593 vdd vdd pch w=2u l=180n
M1452 nw132 t593 0 0 nch w=1u l=180n
Cnw132 nw132 0 2f
CT595 t595 0 0.1f
CT596 t596 0 0.1f
CT597 t597 0 0.1f
M1453 t595 nq66 vdd vdd pch w=2u l=180n
M1454 t595 nw132 vdd vdd pch w=2u l=180n
CT598 t598 0 0.1f
M1455 t595 nq66 t598 0 nch w=1u l=180n
M1456 t598 nw132 0 0 nch w=1u l=180n
M1457 t596 nq66 vdd vdd pch w=2u l=180n
M1458 t596 t595 vdd vdd pch w=2u l=180n
CT599 t599 0 0.1f
M1459 t596 nq66 t599 0 nch w=1u l=180n
M1460 t599 t595 0 0 nch w=1u l=180n
M1461 t597 nw132 vdd vdd pch w=2u l=180n
M1462 t597 t595 vdd vdd pch w=2u l=180n
CT600 t600 0 0.1f
M1463 t597 nw132 t600 0 nch w=1u l=180n
M1464 t600 t595 0 0 nch w=1u l=180n
M1465 nw133 t596 vdd vdd pch w=2u l=180n
M1466 nw133 t597 vdd vdd pch w=2u l=180n
CT601 t601 0 0.1f
M1467 nw133 t596 t601 0 nch w=1u l=180n
M1468 t601 t597 0 0 nch w=1u l=180n
Cnw133 nw133 0 2f
CT602 t602 0 0.1f
M1469 t602 nw132 vdd vdd pch w=2u l=180n
M1470 t602 nq66 vdd vdd pch w=2u l=180n
CT603 t603 0 0.1f
M1471 t602 nw132 t603 0 nch w=1u l=180n
M1472 t603 nq66 0 0 nch w=1u l=180n
M1473 nw134 t602 vdd vdd pch w=2u l=180n
M1474 nw134 t602 0 0 nch w=1u l=180n
Cnw134 nw134 0 2f
CT604 t604 0 0.1f
CT605 t605 0 0.1f
CT606 t606 0 0.1f
M1475 t604 nq67 vdd vdd pch w=2u l=180n
M1476 t604 nw134 vdd vdd pch w=2u l=180n
CT607 t607 0 0.1f
M1477 t604 nq67 t607 0 nch w=1u l=180n
M1478 t607 nw134 0 0 nch w=1u l=180n
M1479 t605 nq67 vdd vdd pch w=2u l=180n
M1480 t605 t604 vdd vdd pch w=2u l=180n
CT608 t608 0 0.1f
M1481 t605 nq67 t608 0 nch w=1u l=180n
M1482 t608 t604 0 0 nch w=1u l=180n
M1483 t606 nw134 vdd vdd pch w=2u l=180n
M1484 t606 t604 vdd vdd pch w=2u l=180n
CT609 t609 0 0.1f
M1485 t606 nw134 t609 0 nch w=1u l=180n
M1486 t609 t604 0 0 nch w=1u l=180n
M1487 nw135 t605 vdd vdd pch w=2u l=180n
M1488 nw135 t606 vdd vdd pch w=2u l=180n
CT610 t610 0 0.1f
M1489 nw135 t605 t610 0 nch w=1u l=180n
M1490 t610 t606 0 0 nch w=1u l=180n
Cnw135 nw135 0 2f
CT611 t611 0 0.1f
M1491 t611 nw134 vdd vdd pch w=2u l=180n
M1492 t611 nq67 vdd vdd pch w=2u l=180n
CT612 t612 0 0.1f
M1493 t611 nw134 t612 0 nch w=1u l=180n
M1494 t612 nq67 0 0 nch w=1u l=180n
M1495 nw136 t611 vdd vdd pch w=2u l=180n
M1496 nw136 t611 0 0 nch w=1u l=180n
Cnw136 nw136 0 2f
CT613 t613 0 0.1f
CT614 t614 0 0.1f
CT615 t615 0 0.1f
M1497 t613 nq68 vdd vdd pch w=2u l=180n
M1498 t613 nw136 vdd vdd pch w=2u l=180n
CT616 t616 0 0.1f
M1499 t613 nq68 t616 0 nch w=1u l=180n
M1500 t616 nw136 0 0 nch w=1u l=180n
M1501 t614 nq68 vdd vdd pch w=2u l=180n
M1502 t614 t613 vdd vdd pch w=2u l=180n
CT617 t617 0 0.1f
M1503 t614 nq68 t617 0 nch w=1u l=180n
M1504 t617 t613 0 0 nch w=1u l=180n
M1505 t615 nw136 vdd vdd pch w=2u l=180n
M1506 t615 t613 vdd vdd pch w=2u l=180n
CT618 t618 0 0.1f
M1507 t615 nw136 t618 0 nch w=1u l=180n
M1508 t618 t613 0 0 nch w=1u l=180n
M1509 nw137 t614 vdd vdd pch w=2u l=180n
M1510 nw137 t615 vdd vdd pch w=2u l=180n
CT619 t619 0 0.1f
M1511 nw137 t614 t619 0 nch w=1u l=180n
M1512 t619 t615 0 0 nch w=1u l=180n
Cnw137 nw137 0 2f
CT620 t620 0 0.1f
M1513 t620 nw136 vdd vdd pch w=2u l=180n
M1514 t620 nq68 vdd vdd pch w=2u l=180n
CT621 t621 0 0.1f
M1515 t620 nw136 t621 0 nch w=1u l=180n
M1516 t621 nq68 0 0 nch w=1u l=180n
M1517 nw138 t620 vdd vdd pch w=2u l=180n
M1518 nw138 t620 0 0 nch w=1u l=180n
Cnw138 nw138 0 2f
CT622 t622 0 0.1f
CT623 t623 0 0.1f
CT624 t624 0 0.1f
M1519 t622 nq69 vdd vdd pch w=2u l=180n
M1520 t622 nw138 vdd vdd pch w=2u l=180n
CT625 t625 0 0.1f
M1521 t622 nq69 t625 0 nch w=1u l=180n
M1522 t625 nw138 0 0 nch w=1u l=180n
M1523 t623 nq69 vdd vdd pch w=2u l=180n
M1524 t623 t622 vdd vdd pch w=2u l=180n
CT626 t626 0 0.1f
M1525 t623 nq69 t626 0 nch w=1u l=180n
M1526 t626 t622 0 0 nch w=1u l=180n
M1527 t624 nw138 vdd vdd pch w=2u l=180n
M1528 t624 t622 vdd vdd pch w=2u l=180n
CT627 t627 0 0.1f
M1529 t624 nw138 t627 0 nch w=1u l=180n
M1530 t627 t622 0 0 nch w=1u l=180n
M1531 nw139 t623 vdd vdd pch w=2u l=180n
M1532 nw139 t624 vdd vdd pch w=2u l=180n
CT628 t628 0 0.1f
M1533 nw139 t623 t628 0 nch w=1u l=180n
M1534 t628 t624 0 0 nch w=1u l=180n
Cnw139 nw139 0 2f
CT629 t629 0 0.1f
M1535 t629 nw138 vdd vdd pch w=2u l=180n
M1536 t629 nq69 vdd vdd pch w=2u l=180n
CT630 t630 0 0.1f
M1537 t629 nw138 t630 0 nch w=1u l=180n
M1538 t630 nq69 0 0 nch w=1u l=180n
M1539 nw140 t629 vdd vdd pch w=2u l=180n
M1540 nw140 t629 0 0 nch w=1u l=180n
Cnw140 nw140 0 2f
CT631 t631 0 0.1f
CT632 t632 0 0.1f
CT633 t633 0 0.1f
M1541 t631 nq70 vdd vdd pch w=2u l=180n
M1542 t631 nw140 vdd vdd pch w=2u l=180n
CT634 t634 0 0.1f
M1543 t631 nq70 t634 0 nch w=1u l=180n
M1544 t634 nw140 0 0 nch w=1u l=180n
M1545 t632 nq70 vdd vdd pch w=2u l=180n
M1546 t632 t631 vdd vdd pch w=2u l=180n
CT635 t635 0 0.1f
M1547 t632 nq70 t635 0 nch w=1u l=180n
M1548 t635 t631 0 0 nch w=1u l=180n
M1549 t633 nw140 vdd vdd pch w=2u l=180n
M1550 t633 t631 vdd vdd pch w=2u l=180n
CT636 t636 0 0.1f
M1551 t633 nw140 t636 0 nch w=1u l=180n
M1552 t636 t631 0 0 nch w=1u l=180n
M1553 nw141 t632 vdd vdd pch w=2u l=180n
M1554 nw141 t633 vdd vdd pch w=2u l=180n
CT637 t637 0 0.1f
M1555 nw141 t632 t637 0 nch w=1u l=180n
M1556 t637 t633 0 0 nch w=1u l=180n
Cnw141 nw141 0 2f
CT638 t638 0 0.1f
M1557 t638 nw140 vdd vdd pch w=2u l=180n
M1558 t638 nq70 vdd vdd pch w=2u l=180n
CT639 t639 0 0.1f
M1559 t638 nw140 t639 0 nch w=1u l=180n
M1560 t639 nq70 0 0 nch w=1u l=180n
M1561 nw142 t638 vdd vdd pch w=2u l=180n
M1562 nw142 t638 0 0 nch w=1u l=180n
Cnw142 nw142 0 2f
CT640 t640 0 0.1f
CT641 t641 0 0.1f
CT642 t642 0 0.1f
M1563 t640 nq71 vdd vdd pch w=2u l=180n
M1564 t640 nw142 vdd vdd pch w=2u l=180n
CT643 t643 0 0.1f
M1565 t640 nq71 t643 0 nch w=1u l=180n
M1566 t643 nw142 0 0 nch w=1u l=180n
M1567 t641 nq71 vdd vdd pch w=2u l=180n
M1568 t641 t640 vdd vdd pch w=2u l=180n
CT644 t644 0 0.1f
M1569 t641 nq71 t644 0 nch w=1u l=180n
M1570 t644 t640 0 0 nch w=1u l=180n
M1571 t642 nw142 vdd vdd pch w=2u l=180n
M1572 t642 t640 vdd vdd pch w=2u l=180n
CT645 t645 0 0.1f
M1573 t642 nw142 t645 0 nch w=1u l=180n
M1574 t645 t640 0 0 nch w=1u l=180n
M1575 nw143 t641 vdd vdd pch w=2u l=180n
M1576 nw143 t642 vdd vdd pch w=2u l=180n
CT646 t646 0 0.1f
M1577 nw143 t641 t646 0 nch w=1u l=180n
M1578 t646 t642 0 0 nch w=1u l=180n
Cnw143 nw143 0 2f
CT647 t647 0 0.1f
M1579 t647 nw142 vdd vdd pch w=2u l=180n
M1580 t647 nq71 vdd vdd pch w=2u l=180n
CT648 t648 0 0.1f
M1581 t647 nw142 t648 0 nch w=1u l=180n
M1582 t648 nq71 0 0 nch w=1u l=180n
M1583 nw144 t647 vdd vdd pch w=2u l=180n
M1584 nw144 t647 0 0 nch w=1u l=180n
Cnw144 nw144 0 2f
CT649 t649 0 0.1f
CT650 t650 0 0.1f
CT651 t651 0 0.1f
M1585 t649 nq72 vdd vdd pch w=2u l=180n
M1586 t649 nw144 vdd vdd pch w=2u l=180n
CT652 t652 0 0.1f
M1587 t649 nq72 t652 0 nch w=1u l=180n
M1588 t652 nw144 0 0 nch w=1u l=180n
M1589 t650 nq72 vdd vdd pch w=2u l=180n
M1590 t650 t649 vdd vdd pch w=2u l=180n
CT653 t653 0 0.1f
M1591 t650 nq72 t653 0 nch w=1u l=180n
M1592 t653 t649 0 0 nch w=1u l=180n
M1593 t651 nw144 vdd vdd pch w=2u l=180n
M1594 t651 t649 vdd vdd pch w=2u l=180n
CT654 t654 0 0.1f
M1595 t651 nw144 t654 0 nch w=1u l=180n
M1596 t654 t649 0 0 nch w=1u l=180n
M1597 nw145 t650 vdd vdd pch w=2u l=180n
M1598 nw145 t651 vdd vdd pch w=2u l=180n
CT655 t655 0 0.1f
M1599 nw145 t650 t655 0 nch w=1u l=180n
M1600 t655 t651 0 0 nch w=1u l=180n
Cnw145 nw145 0 2f
CT656 t656 0 0.1f
M1601 t656 nw144 vdd vdd pch w=2u l=180n
M1602 t656 nq72 vdd vdd pch w=2u l=180n
CT657 t657 0 0.1f
M1603 t656 nw144 t657 0 nch w=1u l=180n
M1604 t657 nq72 0 0 nch w=1u l=180n
M1605 nw146 t656 vdd vdd pch w=2u l=180n
M1606 nw146 t656 0 0 nch w=1u l=180n
Cnw146 nw146 0 2f
CT658 t658 0 0.1f
CT659 t659 0 0.1f
CT660 t660 0 0.1f
M1607 t658 nq73 vdd vdd pch w=2u l=180n
M1608 t658 nw146 vdd vdd pch w=2u l=180n
CT661 t661 0 0.1f
M1609 t658 nq73 t661 0 nch w=1u l=180n
M1610 t661 nw146 0 0 nch w=1u l=180n
M1611 t659 nq73 vdd vdd pch w=2u l=180n
M1612 t659 t658 vdd vdd pch w=2u l=180n
CT662 t662 0 0.1f
M1613 t659 nq73 t662 0 nch w=1u l=180n
M1614 t662 t658 0 0 nch w=1u l=180n
M1615 t660 nw146 vdd vdd pch w=2u l=180n
M1616 t660 t658 vdd vdd pch w=2u l=180n
CT663 t663 0 0.1f
M1617 t660 nw146 t663 0 nch w=1u l=180n
M1618 t663 t658 0 0 nch w=1u l=180n
M1619 nw147 t659 vdd vdd pch w=2u l=180n
M1620 nw147 t660 vdd vdd pch w=2u l=180n
CT664 t664 0 0.1f
M1621 nw147 t659 t664 0 nch w=1u l=180n
M1622 t664 t660 0 0 nch w=1u l=180n
Cnw147 nw147 0 2f
CT665 t665 0 0.1f
M1623 t665 nw146 vdd vdd pch w=2u l=180n
M1624 t665 nq73 vdd vdd pch w=2u l=180n
CT666 t666 0 0.1f
M1625 t665 nw146 t666 0 nch w=1u l=180n
M1626 t666 nq73 0 0 nch w=1u l=180n
M1627 nw148 t665 vdd vdd pch w=2u l=180n
M1628 nw148 t665 0 0 nch w=1u l=180n
Cnw148 nw148 0 2f
M1629 nw149 nq1 vdd vdd pch w=2u l=180n
M1630 nw149 nq3 vdd vdd pch w=2u l=180n
CT667 t667 0 0.1f
M1631 nw149 nq1 t667 0 nch w=1u l=180n
M1632 t667 nq3 0 0 nch w=1u l=180n
Cnw149 nw149 0 2f
M1633 nw150 nq8 0 0 nch w=1u l=180n
M1634 nw150 nq14 0 0 nch w=1u l=180n
CT668 t668 0 0.1f
M1635 t668 nq8 vdd vdd pch w=2u l=180n
M1636 nw150 nq14 t668 vdd pch w=2u l=180n
Cnw150 nw150 0 2f
CT669 t669 0 0.1f
M1637 t669 nq15 vdd vdd pch w=2u l=180n
M1638 t669 nq25 vdd vdd pch w=2u l=180n
CT670 t670 0 0.1f
M1639 t669 nq15 t670 0 nch w=1u l=180n
M1640 t670 nq25 0 0 nch w=1u l=180n
M1641 nw151 t669 vdd vdd pch w=2u l=180n
M1642 nw151 t669 0 0 nch w=1u l=180n
Cnw151 nw151 0 2f
CT671 t671 0 0.1f
M1643 t671 nq22 0 0 nch w=1u l=180n
M1644 t671 nq36 0 0 nch w=1u l=180n
CT672 t672 0 0.1f
M1645 t672 nq22 vdd vdd pch w=2u l=180n
M1646 t671 nq36 t672 vdd pch w=2u l=180n
M1647 nw152 t671 vdd vdd pch w=2u l=180n
M1648 nw152 t671 0 0 nch w=1u l=180n
Cnw152 nw152 0 2f
CT673 t673 0 0.1f
CT674 t674 0 0.1f
CT675 t675 0 0.1f
M1649 t673 nq29 vdd vdd pch w=2u l=180n
M1650 t673 nq47 vdd vdd pch w=2u l=180n
CT676 t676 0 0.1f
M1651 t673 nq29 t676 0 nch w=1u l=180n
M1652 t676 nq47 0 0 nch w=1u l=180n
M1653 t674 nq29 vdd vdd pch w=2u l=180n
M1654 t674 t673 vdd vdd pch w=2u l=180n
CT677 t677 0 0.1f
M1655 t674 nq29 t677 0 nch w=1u l=180n
M1656 t677 t673 0 0 nch w=1u l=180n
M1657 t675 nq47 vdd vdd pch w=2u l=180n
M1658 t675 t673 vdd vdd pch w=2u l=180n
CT678 t678 0 0.1f
M1659 t675 nq47 t678 0 nch w=1u l=180n
M1660 t678 t673 0 0 nch w=1u l=180n
M1661 nw153 t674 vdd vdd pch w=2u l=180n
M1662 nw153 t675 vdd vdd pch w=2u l=180n
CT679 t679 0 0.1f
M1663 nw153 t674 t679 0 nch w=1u l=180n
M1664 t679 t675 0 0 nch w=1u l=180n
Cnw153 nw153 0 2f
M1665 nw154 nq36 vdd vdd pch w=2u l=180n
M1666 nw154 nq58 vdd vdd pch w=2u l=180n
CT680 t680 0 0.1f
M1667 nw154 nq36 t680 0 nch w=1u l=180n
M1668 t680 nq58 0 0 nch w=1u l=180n
Cnw154 nw154 0 2f
M1669 nw155 nq43 0 0 nch w=1u l=180n
M1670 nw155 nq69 0 0 nch w=1u l=180n
CT681 t681 0 0.1f
M1671 t681 nq43 vdd vdd pch w=2u l=180n
M1672 nw155 nq69 t681 vdd pch w=2u l=180n
Cnw155 nw155 0 2f
CT682 t682 0 0.1f
M1673 t682 nq50 vdd vdd pch w=2u l=180n
M1674 t682 ni6 vdd vdd pch w=2u l=180n
CT683 t683 0 0.1f
M1675 t682 nq50 t683 0 nch w=1u l=180n
M1676 t683 ni6 0 0 nch w=1u l=180n
M1677 nw156 t682 vdd vdd pch w=2u l=180n
M1678 nw156 t682 0 0 nch w=1u l=180n
Cnw156 nw156 0 2f
CT684 t684 0 0.1f
M1679 t684 nq57 0 0 nch w=1u l=180n
M1680 t684 nw150 0 0 nch w=1u l=180n
CT685 t685 0 0.1f
M1681 t685 nq57 vdd vdd pch w=2u l=180n
M1682 t684 nw150 t685 vdd pch w=2u l=180n
M1683 nw157 t684 vdd vdd pch w=2u l=180n
M1684 nw157 t684 0 0 nch w=1u l=180n
Cnw157 nw157 0 2f
CT686 t686 0 0.1f
CT687 t687 0 0.1f
CT688 t688 0 0.1f
M1685 t686 nq64 vdd vdd pch w=2u l=180n
M1686 t686 nq3 vdd vdd pch w=2u l=180n
CT689 t689 0 0.1f
M1687 t686 nq64 t689 0 nch w=1u l=180n
M1688 t689 nq3 0 0 nch w=1u l=180n
M1689 t687 nq64 vdd vdd pch w=2u l=180n
M1690 t687 t686 vdd vdd pch w=2u l=180n
CT690 t690 0 0.1f
M1691 t687 nq64 t690 0 nch w=1u l=180n
M1692 t690 t686 0 0 nch w=1u l=180n
M1693 t688 nq3 vdd vdd pch w=2u l=180n
M1694 t688 t686 vdd vdd pch w=2u l=180n
CT691 t691 0 0.1f
M1695 t688 nq3 t691 0 nch w=1u l=180n
M1696 t691 t686 0 0 nch w=1u l=180n
M1697 nw158 t687 vdd vdd pch w=2u l=180n
M1698 nw158 t688 vdd vdd pch w=2u l=180n
CT692 t692 0 0.1f
M1699 nw158 t687 t692 0 nch w=1u l=180n
M1700 t692 t688 0 0 nch w=1u l=180n
Cnw158 nw158 0 2f
M1701 nw159 nq71 vdd vdd pch w=2u l=180n
M1702 nw159 nq13 vdd vdd pch w=2u l=180n
CT693 t693 0 0.1f
M1703 nw159 nq71 t693 0 nch w=1u l=180n
M1704 t693 nq13 0 0 nch w=1u l=180n
Cnw159 nw159 0 2f
M1705 nw160 ni4 0 0 nch w=1u l=180n
M1706 nw160 nq23 0 0 nch w=1u l=180n
CT694 t694 0 0.1f
M1707 t694 ni4 vdd vdd pch w=2u l=180n
M1708 nw160 nq23 t694 vdd pch w=2u l=180n
Cnw160 nw160 0 2f
CT695 t695 0 0.1f
M1709 t695 ni11 vdd vdd pch w=2u l=180n
M1710 t695 nq33 vdd vdd pch w=2u l=180n
CT696 t696 0 0.1f
M1711 t695 ni11 t696 0 nch w=1u l=180n
M1712 t696 nq33 0 0 nch w=1u l=180n
M1713 nw161 t695 vdd vdd pch w=2u l=180n
M1714 nw161 t695 0 0 nch w=1u l=180n
Cnw161 nw161 0 2f
CT697 t697 0 0.1f
M1715 t697 nw151 0 0 nch w=1u l=180n
M1716 t697 nq43 0 0 nch w=1u l=180n
CT698 t698 0 0.1f
M1717 t698 nw151 vdd vdd pch w=2u l=180n
M1718 t697 nq43 t698 vdd pch w=2u l=180n
M1719 nw162 t697 vdd vdd pch w=2u l=180n
M1720 nw162 t697 0 0 nch w=1u l=180n
Cnw162 nw162 0 2f
CT699 t699 0 0.1f
CT700 t700 0 0.1f
CT701 t701 0 0.1f
M1721 t699 nw158 vdd vdd pch w=2u l=180n
M1722 t699 nq53 vdd vdd pch w=2u l=180n
CT702 t702 0 0.1f
M1723 t699 nw158 t702 0 nch w=1u l=180n
M1724 t702 nq53 0 0 nch w=1u l=180n
M1725 t700 nw158 vdd vdd pch w=2u l=180n
M1726 t700 t699 vdd vdd pch w=2u l=180n
CT703 t703 0 0.1f
M1727 t700 nw158 t703 0 nch w=1u l=180n
M1728 t703 t699 0 0 nch w=1u l=180n
M1729 t701 nq53 vdd vdd pch w=2u l=180n
M1730 t701 t699 vdd vdd pch w=2u l=180n
CT704 t704 0 0.1f
M1731 t701 nq53 t704 0 nch w=1u l=180n
M1732 t704 t699 0 0 nch w=1u l=180n
M1733 nw163 t700 vdd vdd pch w=2u l=180n
M1734 nw163 t701 vdd vdd pch w=2u l=180n
CT705 t705 0 0.1f
M1735 nw163 t700 t705 0 nch w=1u l=180n
M1736 t705 t701 0 0 nch w=1u l=180n
Cnw163 nw163 0 2f
M1737 nw164 nq1 vdd vdd pch w=2u l=180n
M1738 nw164 nq63 vdd vdd pch w=2u l=180n
CT706 t706 0 0.1f
M1739 nw164 nq1 t706 0 nch w=1u l=180n
M1740 t706 nq63 0 0 nch w=1u l=180n
Cnw164 nw164 0 2f
M1741 nw165 nq7 0 0 nch w=1u l=180n
M1742 nw165 nq73 0 0 nch w=1u l=180n
CT707 t707 0 0.1f
M1743 t707 nq7 vdd vdd pch w=2u l=180n
M1744 nw165 nq73 t707 vdd pch w=2u l=180n
Cnw165 nw165 0 2f
CT708 t708 0 0.1f
M1745 t708 nq13 vdd vdd pch w=2u l=180n
M1746 t708 ni9 vdd vdd pch w=2u l=180n
CT709 t709 0 0.1f
M1747 t708 nq13 t709 0 nch w=1u l=180n
M1748 t709 ni9 0 0 nch w=1u l=180n
M1749 nw166 t708 vdd vdd pch w=2u l=180n
M1750 nw166 t708 0 0 nch w=1u l=180n
Cnw166 nw166 0 2f
CT710 t710 0 0.1f
M1751 t710 nq19 0 0 nch w=1u l=180n
M1752 t710 nw152 0 0 nch w=1u l=180n
CT711 t711 0 0.1f
M1753 t711 nq19 vdd vdd pch w=2u l=180n
M1754 t710 nw152 t711 vdd pch w=2u l=180n
M1755 nw167 t710 vdd vdd pch w=2u l=180n
M1756 nw167 t710 0 0 nch w=1u l=180n
Cnw167 nw167 0 2f
CT712 t712 0 0.1f
CT713 t713 0 0.1f
CT714 t714 0 0.1f
M1757 t712 nq25 vdd vdd pch w=2u l=180n
M1758 t712 nw162 vdd vdd pch w=2u l=180n
CT715 t715 0 0.1f
M1759 t712 nq25 t715 0 nch w=1u l=180n
M1760 t715 nw162 0 0 nch w=1u l=180n
M1761 t713 nq25 vdd vdd pch w=2u l=180n
M1762 t713 t712 vdd vdd pch w=2u l=180n
CT716 t716 0 0.1f
M1763 t713 nq25 t716 0 nch w=1u l=180n
M1764 t716 t712 0 0 nch w=1u l=180n
M1765 t714 nw162 vdd vdd pch w=2u l=180n
M1766 t714 t712 vdd vdd pch w=2u l=180n
CT717 t717 0 0.1f
M1767 t714 nw162 t717 0 nch w=1u l=180n
M1768 t717 t712 0 0 nch w=1u l=180n
M1769 nw168 t713 vdd vdd pch w=2u l=180n
M1770 nw168 t714 vdd vdd pch w=2u l=180n
CT718 t718 0 0.1f
M1771 nw168 t713 t718 0 nch w=1u l=180n
M1772 t718 t714 0 0 nch w=1u l=180n
Cnw168 nw168 0 2f
M1773 nw169 nq31 vdd vdd pch w=2u l=180n
M1774 nw169 nq3 vdd vdd pch w=2u l=180n
CT719 t719 0 0.1f
M1775 nw169 nq31 t719 0 nch w=1u l=180n
M1776 t719 nq3 0 0 nch w=1u l=180n
Cnw169 nw169 0 2f
M1777 nw170 nq37 0 0 nch w=1u l=180n
M1778 nw170 nq12 0 0 nch w=1u l=180n
CT720 t720 0 0.1f
M1779 t720 nq37 vdd vdd pch w=2u l=180n
M1780 nw170 nq12 t720 vdd pch w=2u l=180n
Cnw170 nw170 0 2f
CT721 t721 0 0.1f
M1781 t721 nq43 vdd vdd pch w=2u l=180n
M1782 t721 nq21 vdd vdd pch w=2u l=180n
CT722 t722 0 0.1f
M1783 t721 nq43 t722 0 nch w=1u l=180n
M1784 t722 nq21 0 0 nch w=1u l=180n
M1785 nw171 t721 vdd vdd pch w=2u l=180n
M1786 nw171 t721 0 0 nch w=1u l=180n
Cnw171 nw171 0 2f
CT723 t723 0 0.1f
M1787 t723 nq49 0 0 nch w=1u l=180n
M1788 t723 nq30 0 0 nch w=1u l=180n
CT724 t724 0 0.1f
M1789 t724 nq49 vdd vdd pch w=2u l=180n
M1790 t723 nq30 t724 vdd pch w=2u l=180n
M1791 nw172 t723 vdd vdd pch w=2u l=180n
M1792 nw172 t723 0 0 nch w=1u l=180n
Cnw172 nw172 0 2f
CT725 t725 0 0.1f
CT726 t726 0 0.1f
CT727 t727 0 0.1f
M1793 t725 nq55 vdd vdd pch w=2u l=180n
M1794 t725 nq39 vdd vdd pch w=2u l=180n
CT728 t728 0 0.1f
M1795 t725 nq55 t728 0 nch w=1u l=180n
M1796 t728 nq39 0 0 nch w=1u l=180n
M1797 t726 nq55 vdd vdd pch w=2u l=180n
M1798 t726 t725 vdd vdd pch w=2u l=180n
CT729 t729 0 0.1f
M1799 t726 nq55 t729 0 nch w=1u l=180n
M1800 t729 t725 0 0 nch w=1u l=180n
M1801 t727 nq39 vdd vdd pch w=2u l=180n
M1802 t727 t725 vdd vdd pch w=2u l=180n
CT730 t730 0 0.1f
M1803 t727 nq39 t730 0 nch w=1u l=180n
M1804 t730 t725 0 0 nch w=1u l=180n
M1805 nw173 t726 vdd vdd pch w=2u l=180n
M1806 nw173 t727 vdd vdd pch w=2u l=180n
CT731 t731 0 0.1f
M1807 nw173 t726 t731 0 nch w=1u l=180n
M1808 t731 t727 0 0 nch w=1u l=180n
Cnw173 nw173 0 2f
M1809 nw174 nq61 vdd vdd pch w=2u l=180n
M1810 nw174 nq48 vdd vdd pch w=2u l=180n
CT732 t732 0 0.1f
M1811 nw174 nq61 t732 0 nch w=1u l=180n
M1812 t732 nq48 0 0 nch w=1u l=180n
Cnw174 nw174 0 2f
M1813 nw175 nq67 0 0 nch w=1u l=180n
M1814 nw175 nq57 0 0 nch w=1u l=180n
CT733 t733 0 0.1f
M1815 t733 nq67 vdd vdd pch w=2u l=180n
M1816 nw175 nq57 t733 vdd pch w=2u l=180n
Cnw175 nw175 0 2f
CT734 t734 0 0.1f
M1817 t734 nq73 vdd vdd pch w=2u l=180n
M1818 t734 nq66 vdd vdd pch w=2u l=180n
CT735 t735 0 0.1f
M1819 t734 nq73 t735 0 nch w=1u l=180n
M1820 t735 nq66 0 0 nch w=1u l=180n
M1821 nw176 t734 vdd vdd pch w=2u l=180n
M1822 nw176 t734 0 0 nch w=1u l=180n
Cnw176 nw176 0 2f
CT736 t736 0 0.1f
M1823 t736 ni5 0 0 nch w=1u l=180n
M1824 t736 ni1 0 0 nch w=1u l=180n
CT737 t737 0 0.1f
M1825 t737 ni5 vdd vdd pch w=2u l=180n
M1826 t736 ni1 t737 vdd pch w=2u l=180n
M1827 nw177 t736 vdd vdd pch w=2u l=180n
M1828 nw177 t736 0 0 nch w=1u l=180n
Cnw177 nw177 0 2f
CT738 t738 0 0.1f
CT739 t739 0 0.1f
CT740 t740 0 0.1f
M1829 t738 ni11 vdd vdd pch w=2u l=180n
M1830 t738 ni10 vdd vdd pch w=2u l=180n
CT741 t741 0 0.1f
M1831 t738 ni11 t741 0 nch w=1u l=180n
M1832 t741 ni10 0 0 nch w=1u l=180n
M1833 t739 ni11 vdd vdd pch w=2u l=180n
M1834 t739 t738 vdd vdd pch w=2u l=180n
CT742 t742 0 0.1f
M1835 t739 ni11 t742 0 nch w=1u l=180n
M1836 t742 t738 0 0 nch w=1u l=180n
M1837 t740 ni10 vdd vdd pch w=2u l=180n
M1838 t740 t738 vdd vdd pch w=2u l=180n
CT743 t743 0 0.1f
M1839 t740 ni10 t743 0 nch w=1u l=180n
M1840 t743 t738 0 0 nch w=1u l=180n
M1841 nw178 t739 vdd vdd pch w=2u l=180n
M1842 nw178 t740 vdd vdd pch w=2u l=180n
CT744 t744 0 0.1f
M1843 nw178 t739 t744 0 nch w=1u l=180n
M1844 t744 t740 0 0 nch w=1u l=180n
Cnw178 nw178 0 2f
M1845 nw179 nw150 vdd vdd pch w=2u l=180n
M1846 nw179 nw152 vdd vdd pch w=2u l=180n
CT745 t745 0 0.1f
M1847 nw179 nw150 t745 0 nch w=1u l=180n
M1848 t745 nw152 0 0 nch w=1u l=180n
Cnw179 nw179 0 2f
M1849 nw180 nw156 0 0 nch w=1u l=180n
M1850 nw180 nw161 0 0 nch w=1u l=180n
CT746 t746 0 0.1f
M1851 t746 nw156 vdd vdd pch w=2u l=180n
M1852 nw180 nw161 t746 vdd pch w=2u l=180n
Cnw180 nw180 0 2f
CT747 t747 0 0.1f
M1853 t747 nw162 vdd vdd pch w=2u l=180n
M1854 t747 nw170 vdd vdd pch w=2u l=180n
CT748 t748 0 0.1f
M1855 t747 nw162 t748 0 nch w=1u l=180n
M1856 t748 nw170 0 0 nch w=1u l=180n
M1857 nw181 t747 vdd vdd pch w=2u l=180n
M1858 nw181 t747 0 0 nch w=1u l=180n
Cnw181 nw181 0 2f
CT749 t749 0 0.1f
M1859 t749 nw168 0 0 nch w=1u l=180n
M1860 t749 nw179 0 0 nch w=1u l=180n
CT750 t750 0 0.1f
M1861 t750 nw168 vdd vdd pch w=2u l=180n
M1862 t749 nw179 t750 vdd pch w=2u l=180n
M1863 nw182 t749 vdd vdd pch w=2u l=180n
M1864 nw182 t749 0 0 nch w=1u l=180n
Cnw182 nw182 0 2f
CT751 t751 0 0.1f
CT752 t752 0 0.1f
CT753 t753 0 0.1f
M1865 t751 nw174 vdd vdd pch w=2u l=180n
M1866 t751 nq5 vdd vdd pch w=2u l=180n
CT754 t754 0 0.1f
M1867 t751 nw174 t754 0 nch w=1u l=180n
M1868 t754 nq5 0 0 nch w=1u l=180n
M1869 t752 nw174 vdd vdd pch w=2u l=180n
M1870 t752 t751 vdd vdd pch w=2u l=180n
CT755 t755 0 0.1f
M1871 t752 nw174 t755 0 nch w=1u l=180n
M1872 t755 t751 0 0 nch w=1u l=180n
M1873 t753 nq5 vdd vdd pch w=2u l=180n
M1874 t753 t751 vdd vdd pch w=2u l=180n
CT756 t756 0 0.1f
M1875 t753 nq5 t756 0 nch w=1u l=180n
M1876 t756 t751 0 0 nch w=1u l=180n
M1877 nw183 t752 vdd vdd pch w=2u l=180n
M1878 nw183 t753 vdd vdd pch w=2u l=180n
CT757 t757 0 0.1f
M1879 nw183 t752 t757 0 nch w=1u l=180n
M1880 t757 t753 0 0 nch w=1u l=180n
Cnw183 nw183 0 2f
M1881 nw184 nw180 vdd vdd pch w=2u l=180n
M1882 nw184 nq13 vdd vdd pch w=2u l=180n
CT758 t758 0 0.1f
M1883 nw184 nw180 t758 0 nch w=1u l=180n
M1884 t758 nq13 0 0 nch w=1u l=180n
Cnw184 nw184 0 2f
M1885 nw185 nq1 0 0 nch w=1u l=180n
M1886 nw185 nq21 0 0 nch w=1u l=180n
CT759 t759 0 0.1f
M1887 t759 nq1 vdd vdd pch w=2u l=180n
M1888 nw185 nq21 t759 vdd pch w=2u l=180n
Cnw185 nw185 0 2f
CT760 t760 0 0.1f
M1889 t760 nq6 vdd vdd pch w=2u l=180n
M1890 t760 nq29 vdd vdd pch w=2u l=180n
CT761 t761 0 0.1f
M1891 t760 nq6 t761 0 nch w=1u l=180n
M1892 t761 nq29 0 0 nch w=1u l=180n
M1893 nw186 t760 vdd vdd pch w=2u l=180n
M1894 nw186 t760 0 0 nch w=1u l=180n
Cnw186 nw186 0 2f
CT762 t762 0 0.1f
M1895 t762 nq11 0 0 nch w=1u l=180n
M1896 t762 nq37 0 0 nch w=1u l=180n
CT763 t763 0 0.1f
M1897 t763 nq11 vdd vdd pch w=2u l=180n
M1898 t762 nq37 t763 vdd pch w=2u l=180n
M1899 nw187 t762 vdd vdd pch w=2u l=180n
M1900 nw187 t762 0 0 nch w=1u l=180n
Cnw187 nw187 0 2f
CT764 t764 0 0.1f
CT765 t765 0 0.1f
CT766 t766 0 0.1f
M1901 t764 nq16 vdd vdd pch w=2u l=180n
M1902 t764 nq45 vdd vdd pch w=2u l=180n
CT767 t767 0 0.1f
M1903 t764 nq16 t767 0 nch w=1u l=180n
M1904 t767 nq45 0 0 nch w=1u l=180n
M1905 t765 nq16 vdd vdd pch w=2u l=180n
M1906 t765 t764 vdd vdd pch w=2u l=180n
CT768 t768 0 0.1f
M1907 t765 nq16 t768 0 nch w=1u l=180n
M1908 t768 t764 0 0 nch w=1u l=180n
M1909 t766 nq45 vdd vdd pch w=2u l=180n
M1910 t766 t764 vdd vdd pch w=2u l=180n
CT769 t769 0 0.1f
M1911 t766 nq45 t769 0 nch w=1u l=180n
M1912 t769 t764 0 0 nch w=1u l=180n
M1913 nw188 t765 vdd vdd pch w=2u l=180n
M1914 nw188 t766 vdd vdd pch w=2u l=180n
CT770 t770 0 0.1f
M1915 nw188 t765 t770 0 nch w=1u l=180n
M1916 t770 t766 0 0 nch w=1u l=180n
Cnw188 nw188 0 2f
M1917 nw189 nq21 vdd vdd pch w=2u l=180n
M1918 nw189 nq53 vdd vdd pch w=2u l=180n
CT771 t771 0 0.1f
M1919 nw189 nq21 t771 0 nch w=1u l=180n
M1920 t771 nq53 0 0 nch w=1u l=180n
Cnw189 nw189 0 2f
M1921 nw190 nq26 0 0 nch w=1u l=180n
M1922 nw190 nq61 0 0 nch w=1u l=180n
CT772 t772 0 0.1f
M1923 t772 nq26 vdd vdd pch w=2u l=180n
M1924 nw190 nq61 t772 vdd pch w=2u l=180n
Cnw190 nw190 0 2f
CT773 t773 0 0.1f
M1925 t773 nq31 vdd vdd pch w=2u l=180n
M1926 t773 nq69 vdd vdd pch w=2u l=180n
CT774 t774 0 0.1f
M1927 t773 nq31 t774 0 nch w=1u l=180n
M1928 t774 nq69 0 0 nch w=1u l=180n
M1929 nw191 t773 vdd vdd pch w=2u l=180n
M1930 nw191 t773 0 0 nch w=1u l=180n
Cnw191 nw191 0 2f
CT775 t775 0 0.1f
M1931 t775 nq36 0 0 nch w=1u l=180n
M1932 t775 ni3 0 0 nch w=1u l=180n
CT776 t776 0 0.1f
M1933 t776 nq36 vdd vdd pch w=2u l=180n
M1934 t775 ni3 t776 vdd pch w=2u l=180n
M1935 nw192 t775 vdd vdd pch w=2u l=180n
M1936 nw192 t775 0 0 nch w=1u l=180n
Cnw192 nw192 0 2f
CT777 t777 0 0.1f
CT778 t778 0 0.1f
CT779 t779 0 0.1f
M1937 t777 nq41 vdd vdd pch w=2u l=180n
M1938 t777 ni11 vdd vdd pch w=2u l=180n
CT780 t780 0 0.1f
M1939 t777 nq41 t780 0 nch w=1u l=180n
M1940 t780 ni11 0 0 nch w=1u l=180n
M1941 t778 nq41 vdd vdd pch w=2u l=180n
M1942 t778 t777 vdd vdd pch w=2u l=180n
CT781 t781 0 0.1f
M1943 t778 nq41 t781 0 nch w=1u l=180n
M1944 t781 t777 0 0 nch w=1u l=180n
M1945 t779 ni11 vdd vdd pch w=2u l=180n
M1946 t779 t777 vdd vdd pch w=2u l=180n
CT782 t782 0 0.1f
M1947 t779 ni11 t782 0 nch w=1u l=180n
M1948 t782 t777 0 0 nch w=1u l=180n
M1949 nw193 t778 vdd vdd pch w=2u l=180n
M1950 nw193 t779 vdd vdd pch w=2u l=180n
CT783 t783 0 0.1f
M1951 nw193 t778 t783 0 nch w=1u l=180n
M1952 t783 t779 0 0 nch w=1u l=180n
Cnw193 nw193 0 2f
M1953 nw194 nq46 vdd vdd pch w=2u l=180n
M1954 nw194 nw152 vdd vdd pch w=2u l=180n
CT784 t784 0 0.1f
M1955 nw194 nq46 t784 0 nch w=1u l=180n
M1956 t784 nw152 0 0 nch w=1u l=180n
Cnw194 nw194 0 2f
M1957 nw195 nq51 0 0 nch w=1u l=180n
M1958 nw195 nw160 0 0 nch w=1u l=180n
CT785 t785 0 0.1f
M1959 t785 nq51 vdd vdd pch w=2u l=180n
M1960 nw195 nw160 t785 vdd pch w=2u l=180n
Cnw195 nw195 0 2f
CT786 t786 0 0.1f
M1961 t786 nq56 vdd vdd pch w=2u l=180n
M1962 t786 nw168 vdd vdd pch w=2u l=180n
CT787 t787 0 0.1f
M1963 t786 nq56 t787 0 nch w=1u l=180n
M1964 t787 nw168 0 0 nch w=1u l=180n
M1965 nw196 t786 vdd vdd pch w=2u l=180n
M1966 nw196 t786 0 0 nch w=1u l=180n
Cnw196 nw196 0 2f
CT788 t788 0 0.1f
M1967 t788 nq61 0 0 nch w=1u l=180n
M1968 t788 nw176 0 0 nch w=1u l=180n
CT789 t789 0 0.1f
M1969 t789 nq61 vdd vdd pch w=2u l=180n
M1970 t788 nw176 t789 vdd pch w=2u l=180n
M1971 nw197 t788 vdd vdd pch w=2u l=180n
M1972 nw197 t788 0 0 nch w=1u l=180n
Cnw197 nw197 0 2f
CT790 t790 0 0.1f
CT791 t791 0 0.1f
CT792 t792 0 0.1f
M1973 t790 nq66 vdd vdd pch w=2u l=180n
M1974 t790 nw184 vdd vdd pch w=2u l=180n
CT793 t793 0 0.1f
M1975 t790 nq66 t793 0 nch w=1u l=180n
M1976 t793 nw184 0 0 nch w=1u l=180n
M1977 t791 nq66 vdd vdd pch w=2u l=180n
M1978 t791 t790 vdd vdd pch w=2u l=180n
CT794 t794 0 0.1f
M1979 t791 nq66 t794 0 nch w=1u l=180n
M1980 t794 t790 0 0 nch w=1u l=180n
M1981 t792 nw184 vdd vdd pch w=2u l=180n
M1982 t792 t790 vdd vdd pch w=2u l=180n
CT795 t795 0 0.1f
M1983 t792 nw184 t795 0 nch w=1u l=180n
M1984 t795 t790 0 0 nch w=1u l=180n
M1985 nw198 t791 vdd vdd pch w=2u l=180n
M1986 nw198 t792 vdd vdd pch w=2u l=180n
CT796 t796 0 0.1f
M1987 nw198 t791 t796 0 nch w=1u l=180n
M1988 t796 t792 0 0 nch w=1u l=180n
Cnw198 nw198 0 2f
M1989 nw199 nq71 vdd vdd pch w=2u l=180n
M1990 nw199 nw192 vdd vdd pch w=2u l=180n
CT797 t797 0 0.1f
M1991 nw199 nq71 t797 0 nch w=1u l=180n
M1992 t797 nw192 0 0 nch w=1u l=180n
Cnw199 nw199 0 2f
M1993 nw200 ni2 0 0 nch w=1u l=180n
M1994 nw200 nq0 0 0 nch w=1u l=180n
CT798 t798 0 0.1f
M1995 t798 ni2 vdd vdd pch w=2u l=180n
M1996 nw200 nq0 t798 vdd pch w=2u l=180n
Cnw200 nw200 0 2f
CT799 t799 0 0.1f
M1997 t799 ni7 vdd vdd pch w=2u l=180n
M1998 t799 nq7 vdd vdd pch w=2u l=180n
CT800 t800 0 0.1f
M1999 t799 ni7 t800 0 nch w=1u l=180n
M2000 t800 nq7 0 0 nch w=1u l=180n
M2001 nw201 t799 vdd vdd pch w=2u l=180n
M2002 nw201 t799 0 0 nch w=1u l=180n
Cnw201 nw201 0 2f
CT801 t801 0 0.1f
M2003 t801 ni12 0 0 nch w=1u l=180n
M2004 t801 nq14 0 0 nch w=1u l=180n
CT802 t802 0 0.1f
M2005 t802 ni12 vdd vdd pch w=2u l=180n
M2006 t801 nq14 t802 vdd pch w=2u l=180n
M2007 nw202 t801 vdd vdd pch w=2u l=180n
M2008 nw202 t801 0 0 nch w=1u l=180n
Cnw202 nw202 0 2f
CT803 t803 0 0.1f
CT804 t804 0 0.1f
CT805 t805 0 0.1f
M2009 t803 nw150 vdd vdd pch w=2u l=180n
M2010 t803 nq21 vdd vdd pch w=2u l=180n
CT806 t806 0 0.1f
M2011 t803 nw150 t806 0 nch w=1u l=180n
M2012 t806 nq21 0 0 nch w=1u l=180n
M2013 t804 nw150 vdd vdd pch w=2u l=180n
M2014 t804 t803 vdd vdd pch w=2u l=180n
CT807 t807 0 0.1f
M2015 t804 nw150 t807 0 nch w=1u l=180n
M2016 t807 t803 0 0 nch w=1u l=180n
M2017 t805 nq21 vdd vdd pch w=2u l=180n
M2018 t805 t803 vdd vdd pch w=2u l=180n
CT808 t808 0 0.1f
M2019 t805 nq21 t808 0 nch w=1u l=180n
M2020 t808 t803 0 0 nch w=1u l=180n
M2021 nw203 t804 vdd vdd pch w=2u l=180n
M2022 nw203 t805 vdd vdd pch w=2u l=180n
CT809 t809 0 0.1f
M2023 nw203 t804 t809 0 nch w=1u l=180n
M2024 t809 t805 0 0 nch w=1u l=180n
Cnw203 nw203 0 2f
M2025 nw204 nw155 vdd vdd pch w=2u l=180n
M2026 nw204 nq28 vdd vdd pch w=2u l=180n
CT810 t810 0 0.1f
M2027 nw204 nw155 t810 0 nch w=1u l=180n
M2028 t810 nq28 0 0 nch w=1u l=180n
Cnw204 nw204 0 2f
M2029 nw205 nw160 0 0 nch w=1u l=180n
M2030 nw205 nq35 0 0 nch w=1u l=180n
CT811 t811 0 0.1f
M2031 t811 nw160 vdd vdd pch w=2u l=180n
M2032 nw205 nq35 t811 vdd pch w=2u l=180n
Cnw205 nw205 0 2f
CT812 t812 0 0.1f
M2033 t812 nw165 vdd vdd pch w=2u l=180n
M2034 t812 nq42 vdd vdd pch w=2u l=180n
CT813 t813 0 0.1f
M2035 t812 nw165 t813 0 nch w=1u l=180n
M2036 t813 nq42 0 0 nch w=1u l=180n
M2037 nw206 t812 vdd vdd pch w=2u l=180n
M2038 nw206 t812 0 0 nch w=1u l=180n
Cnw206 nw206 0 2f
CT814 t814 0 0.1f
M2039 t814 nw170 0 0 nch w=1u l=180n
M2040 t814 nq49 0 0 nch w=1u l=180n
CT815 t815 0 0.1f
M2041 t815 nw170 vdd vdd pch w=2u l=180n
M2042 t814 nq49 t815 vdd pch w=2u l=180n
M2043 nw207 t814 vdd vdd pch w=2u l=180n
M2044 nw207 t814 0 0 nch w=1u l=180n
Cnw207 nw207 0 2f
CT816 t816 0 0.1f
CT817 t817 0 0.1f
CT818 t818 0 0.1f
M2045 t816 nw175 vdd vdd pch w=2u l=180n
M2046 t816 nq56 vdd vdd pch w=2u l=180n
CT819 t819 0 0.1f
M2047 t816 nw175 t819 0 nch w=1u l=180n
M2048 t819 nq56 0 0 nch w=1u l=180n
M2049 t817 nw175 vdd vdd pch w=2u l=180n
M2050 t817 t816 vdd vdd pch w=2u l=180n
CT820 t820 0 0.1f
M2051 t817 nw175 t820 0 nch w=1u l=180n
M2052 t820 t816 0 0 nch w=1u l=180n
M2053 t818 nq56 vdd vdd pch w=2u l=180n
M2054 t818 t816 vdd vdd pch w=2u l=180n
CT821 t821 0 0.1f
M2055 t818 nq56 t821 0 nch w=1u l=180n
M2056 t821 t816 0 0 nch w=1u l=180n
M2057 nw208 t817 vdd vdd pch w=2u l=180n
M2058 nw208 t818 vdd vdd pch w=2u l=180n
CT822 t822 0 0.1f
M2059 nw208 t817 t822 0 nch w=1u l=180n
M2060 t822 t818 0 0 nch w=1u l=180n
Cnw208 nw208 0 2f
M2061 nw209 nw180 vdd vdd pch w=2u l=180n
M2062 nw209 nq63 vdd vdd pch w=2u l=180n
CT823 t823 0 0.1f
M2063 nw209 nw180 t823 0 nch w=1u l=180n
M2064 t823 nq63 0 0 nch w=1u l=180n
Cnw209 nw209 0 2f
M2065 nw210 nw185 0 0 nch w=1u l=180n
M2066 nw210 nq70 0 0 nch w=1u l=180n
CT824 t824 0 0.1f
M2067 t824 nw185 vdd vdd pch w=2u l=180n
M2068 nw210 nq70 t824 vdd pch w=2u l=180n
Cnw210 nw210 0 2f
CT825 t825 0 0.1f
M2069 t825 nw190 vdd vdd pch w=2u l=180n
M2070 t825 ni3 vdd vdd pch w=2u l=180n
CT826 t826 0 0.1f
M2071 t825 nw190 t826 0 nch w=1u l=180n
M2072 t826 ni3 0 0 nch w=1u l=180n
M2073 nw211 t825 vdd vdd pch w=2u l=180n
M2074 nw211 t825 0 0 nch w=1u l=180n
Cnw211 nw211 0 2f
CT827 t827 0 0.1f
M2075 t827 nw195 0 0 nch w=1u l=180n
M2076 t827 ni10 0 0 nch w=1u l=180n
CT828 t828 0 0.1f
M2077 t828 nw195 vdd vdd pch w=2u l=180n
M2078 t827 ni10 t828 vdd pch w=2u l=180n
M2079 nw212 t827 vdd vdd pch w=2u l=180n
M2080 nw212 t827 0 0 nch w=1u l=180n
Cnw212 nw212 0 2f
CT829 t829 0 0.1f
CT830 t830 0 0.1f
CT831 t831 0 0.1f
M2081 t829 nw200 vdd vdd pch w=2u l=180n
M2082 t829 nw150 vdd vdd pch w=2u l=180n
CT832 t832 0 0.1f
M2083 t829 nw200 t832 0 nch w=1u l=180n
M2084 t832 nw150 0 0 nch w=1u l=180n
M2085 t830 nw200 vdd vdd pch w=2u l=180n
M2086 t830 t829 vdd vdd pch w=2u l=180n
CT833 t833 0 0.1f
M2087 t830 nw200 t833 0 nch w=1u l=180n
M2088 t833 t829 0 0 nch w=1u l=180n
M2089 t831 nw150 vdd vdd pch w=2u l=180n
M2090 t831 t829 vdd vdd pch w=2u l=180n
CT834 t834 0 0.1f
M2091 t831 nw150 t834 0 nch w=1u l=180n
M2092 t834 t829 0 0 nch w=1u l=180n
M2093 nw213 t830 vdd vdd pch w=2u l=180n
M2094 nw213 t831 vdd vdd pch w=2u l=180n
CT835 t835 0 0.1f
M2095 nw213 t830 t835 0 nch w=1u l=180n
M2096 t835 t831 0 0 nch w=1u l=180n
Cnw213 nw213 0 2f
M2097 nw214 nw205 vdd vdd pch w=2u l=180n
M2098 nw214 nw157 vdd vdd pch w=2u l=180n
CT836 t836 0 0.1f
M2099 nw214 nw205 t836 0 nch w=1u l=180n
M2100 t836 nw157 0 0 nch w=1u l=180n
Cnw214 nw214 0 2f
M2101 nw215 nw210 0 0 nch w=1u l=180n
M2102 nw215 nw164 0 0 nch w=1u l=180n
CT837 t837 0 0.1f
M2103 t837 nw210 vdd vdd pch w=2u l=180n
M2104 nw215 nw164 t837 vdd pch w=2u l=180n
Cnw215 nw215 0 2f
CT838 t838 0 0.1f
M2105 t838 nw215 vdd vdd pch w=2u l=180n
M2106 t838 nw171 vdd vdd pch w=2u l=180n
CT839 t839 0 0.1f
M2107 t838 nw215 t839 0 nch w=1u l=180n
M2108 t839 nw171 0 0 nch w=1u l=180n
M2109 nw216 t838 vdd vdd pch w=2u l=180n
M2110 nw216 t838 0 0 nch w=1u l=180n
Cnw216 nw216 0 2f
CT840 t840 0 0.1f
M2111 t840 nq3 0 0 nch w=1u l=180n
M2112 t840 nw178 0 0 nch w=1u l=180n
CT841 t841 0 0.1f
M2113 t841 nq3 vdd vdd pch w=2u l=180n
M2114 t840 nw178 t841 vdd pch w=2u l=180n
M2115 nw217 t840 vdd vdd pch w=2u l=180n
M2116 nw217 t840 0 0 nch w=1u l=180n
Cnw217 nw217 0 2f
CT842 t842 0 0.1f
CT843 t843 0 0.1f
CT844 t844 0 0.1f
M2117 t842 nq7 vdd vdd pch w=2u l=180n
M2118 t842 nw185 vdd vdd pch w=2u l=180n
CT845 t845 0 0.1f
M2119 t842 nq7 t845 0 nch w=1u l=180n
M2120 t845 nw185 0 0 nch w=1u l=180n
M2121 t843 nq7 vdd vdd pch w=2u l=180n
M2122 t843 t842 vdd vdd pch w=2u l=180n
CT846 t846 0 0.1f
M2123 t843 nq7 t846 0 nch w=1u l=180n
M2124 t846 t842 0 0 nch w=1u l=180n
M2125 t844 nw185 vdd vdd pch w=2u l=180n
M2126 t844 t842 vdd vdd pch w=2u l=180n
CT847 t847 0 0.1f
M2127 t844 nw185 t847 0 nch w=1u l=180n
M2128 t847 t842 0 0 nch w=1u l=180n
M2129 nw218 t843 vdd vdd pch w=2u l=180n
M2130 nw218 t844 vdd vdd pch w=2u l=180n
CT848 t848 0 0.1f
M2131 nw218 t843 t848 0 nch w=1u l=180n
M2132 t848 t844 0 0 nch w=1u l=180n
Cnw218 nw218 0 2f
M2133 nw219 nq11 vdd vdd pch w=2u l=180n
M2134 nw219 nw192 vdd vdd pch w=2u l=180n
CT849 t849 0 0.1f
M2135 nw219 nq11 t849 0 nch w=1u l=180n
M2136 t849 nw192 0 0 nch w=1u l=180n
Cnw219 nw219 0 2f
M2137 nw220 nq15 0 0 nch w=1u l=180n
M2138 nw220 nw199 0 0 nch w=1u l=180n
CT850 t850 0 0.1f
M2139 t850 nq15 vdd vdd pch w=2u l=180n
M2140 nw220 nw199 t850 vdd pch w=2u l=180n
Cnw220 nw220 0 2f
CT851 t851 0 0.1f
M2141 t851 nq19 vdd vdd pch w=2u l=180n
M2142 t851 nw206 vdd vdd pch w=2u l=180n
CT852 t852 0 0.1f
M2143 t851 nq19 t852 0 nch w=1u l=180n
M2144 t852 nw206 0 0 nch w=1u l=180n
M2145 nw221 t851 vdd vdd pch w=2u l=180n
M2146 nw221 t851 0 0 nch w=1u l=180n
Cnw221 nw221 0 2f
CT853 t853 0 0.1f
M2147 t853 nq23 0 0 nch w=1u l=180n
M2148 t853 nw213 0 0 nch w=1u l=180n
CT854 t854 0 0.1f
M2149 t854 nq23 vdd vdd pch w=2u l=180n
M2150 t853 nw213 t854 vdd pch w=2u l=180n
M2151 nw222 t853 vdd vdd pch w=2u l=180n
M2152 nw222 t853 0 0 nch w=1u l=180n
Cnw222 nw222 0 2f
CT855 t855 0 0.1f
CT856 t856 0 0.1f
CT857 t857 0 0.1f
M2153 t855 nq27 vdd vdd pch w=2u l=180n
M2154 t855 nw220 vdd vdd pch w=2u l=180n
CT858 t858 0 0.1f
M2155 t855 nq27 t858 0 nch w=1u l=180n
M2156 t858 nw220 0 0 nch w=1u l=180n
M2157 t856 nq27 vdd vdd pch w=2u l=180n
M2158 t856 t855 vdd vdd pch w=2u l=180n
CT859 t859 0 0.1f
M2159 t856 nq27 t859 0 nch w=1u l=180n
M2160 t859 t855 0 0 nch w=1u l=180n
M2161 t857 nw220 vdd vdd pch w=2u l=180n
M2162 t857 t855 vdd vdd pch w=2u l=180n
CT860 t860 0 0.1f
M2163 t857 nw220 t860 0 nch w=1u l=180n
M2164 t860 t855 0 0 nch w=1u l=180n
M2165 nw223 t856 vdd vdd pch w=2u l=180n
M2166 nw223 t857 vdd vdd pch w=2u l=180n
CT861 t861 0 0.1f
M2167 nw223 t856 t861 0 nch w=1u l=180n
M2168 t861 t857 0 0 nch w=1u l=180n
Cnw223 nw223 0 2f
M2169 nw224 nq31 vdd vdd pch w=2u l=180n
M2170 nw224 nq3 vdd vdd pch w=2u l=180n
CT862 t862 0 0.1f
M2171 nw224 nq31 t862 0 nch w=1u l=180n
M2172 t862 nq3 0 0 nch w=1u l=180n
Cnw224 nw224 0 2f
M2173 nw225 nq35 0 0 nch w=1u l=180n
M2174 nw225 nq9 0 0 nch w=1u l=180n
CT863 t863 0 0.1f
M2175 t863 nq35 vdd vdd pch w=2u l=180n
M2176 nw225 nq9 t863 vdd pch w=2u l=180n
Cnw225 nw225 0 2f
CT864 t864 0 0.1f
M2177 t864 nq39 vdd vdd pch w=2u l=180n
M2178 t864 nq15 vdd vdd pch w=2u l=180n
CT865 t865 0 0.1f
M2179 t864 nq39 t865 0 nch w=1u l=180n
M2180 t865 nq15 0 0 nch w=1u l=180n
M2181 nw226 t864 vdd vdd pch w=2u l=180n
M2182 nw226 t864 0 0 nch w=1u l=180n
Cnw226 nw226 0 2f
CT866 t866 0 0.1f
M2183 t866 nq43 0 0 nch w=1u l=180n
M2184 t866 nq21 0 0 nch w=1u l=180n
CT867 t867 0 0.1f
M2185 t867 nq43 vdd vdd pch w=2u l=180n
M2186 t866 nq21 t867 vdd pch w=2u l=180n
M2187 nw227 t866 vdd vdd pch w=2u l=180n
M2188 nw227 t866 0 0 nch w=1u l=180n
Cnw227 nw227 0 2f
CT868 t868 0 0.1f
CT869 t869 0 0.1f
CT870 t870 0 0.1f
M2189 t868 nq47 vdd vdd pch w=2u l=180n
M2190 t868 nq27 vdd vdd pch w=2u l=180n
CT871 t871 0 0.1f
M2191 t868 nq47 t871 0 nch w=1u l=180n
M2192 t871 nq27 0 0 nch w=1u l=180n
M2193 t869 nq47 vdd vdd pch w=2u l=180n
M2194 t869 t868 vdd vdd pch w=2u l=180n
CT872 t872 0 0.1f
M2195 t869 nq47 t872 0 nch w=1u l=180n
M2196 t872 t868 0 0 nch w=1u l=180n
M2197 t870 nq27 vdd vdd pch w=2u l=180n
M2198 t870 t868 vdd vdd pch w=2u l=180n
CT873 t873 0 0.1f
M2199 t870 nq27 t873 0 nch w=1u l=180n
M2200 t873 t868 0 0 nch w=1u l=180n
M2201 nw228 t869 vdd vdd pch w=2u l=180n
M2202 nw228 t870 vdd vdd pch w=2u l=180n
CT874 t874 0 0.1f
M2203 nw228 t869 t874 0 nch w=1u l=180n
M2204 t874 t870 0 0 nch w=1u l=180n
Cnw228 nw228 0 2f
M2205 nw229 nq51 vdd vdd pch w=2u l=180n
M2206 nw229 nq33 vdd vdd pch w=2u l=180n
CT875 t875 0 0.1f
M2207 nw229 nq51 t875 0 nch w=1u l=180n
M2208 t875 nq33 0 0 nch w=1u l=180n
Cnw229 nw229 0 2f
M2209 nw230 nq55 0 0 nch w=1u l=180n
M2210 nw230 nq39 0 0 nch w=1u l=180n
CT876 t876 0 0.1f
M2211 t876 nq55 vdd vdd pch w=2u l=180n
M2212 nw230 nq39 t876 vdd pch w=2u l=180n
Cnw230 nw230 0 2f
CT877 t877 0 0.1f
M2213 t877 nq59 vdd vdd pch w=2u l=180n
M2214 t877 nq45 vdd vdd pch w=2u l=180n
CT878 t878 0 0.1f
M2215 t877 nq59 t878 0 nch w=1u l=180n
M2216 t878 nq45 0 0 nch w=1u l=180n
M2217 nw231 t877 vdd vdd pch w=2u l=180n
M2218 nw231 t877 0 0 nch w=1u l=180n
Cnw231 nw231 0 2f
CT879 t879 0 0.1f
M2219 t879 nq63 0 0 nch w=1u l=180n
M2220 t879 nq51 0 0 nch w=1u l=180n
CT880 t880 0 0.1f
M2221 t880 nq63 vdd vdd pch w=2u l=180n
M2222 t879 nq51 t880 vdd pch w=2u l=180n
M2223 nw232 t879 vdd vdd pch w=2u l=180n
M2224 nw232 t879 0 0 nch w=1u l=180n
Cnw232 nw232 0 2f
CT881 t881 0 0.1f
CT882 t882 0 0.1f
CT883 t883 0 0.1f
M2225 t881 nq67 vdd vdd pch w=2u l=180n
M2226 t881 nq57 vdd vdd pch w=2u l=180n
CT884 t884 0 0.1f
M2227 t881 nq67 t884 0 nch w=1u l=180n
M2228 t884 nq57 0 0 nch w=1u l=180n
M2229 t882 nq67 vdd vdd pch w=2u l=180n
M2230 t882 t881 vdd vdd pch w=2u l=180n
CT885 t885 0 0.1f
M2231 t882 nq67 t885 0 nch w=1u l=180n
M2232 t885 t881 0 0 nch w=1u l=180n
M2233 t883 nq57 vdd vdd pch w=2u l=180n
M2234 t883 t881 vdd vdd pch w=2u l=180n
CT886 t886 0 0.1f
M2235 t883 nq57 t886 0 nch w=1u l=180n
M2236 t886 t881 0 0 nch w=1u l=180n
M2237 nw233 t882 vdd vdd pch w=2u l=180n
M2238 nw233 t883 vdd vdd pch w=2u l=180n
CT887 t887 0 0.1f
M2239 nw233 t882 t887 0 nch w=1u l=180n
M2240 t887 t883 0 0 nch w=1u l=180n
Cnw233 nw233 0 2f
M2241 nw234 nq71 vdd vdd pch w=2u l=180n
M2242 nw234 nq63 vdd vdd pch w=2u l=180n
CT888 t888 0 0.1f
M2243 nw234 nq71 t888 0 nch w=1u l=180n
M2244 t888 nq63 0 0 nch w=1u l=180n
Cnw234 nw234 0 2f
M2245 nw235 ni1 0 0 nch w=1u l=180n
M2246 nw235 nq69 0 0 nch w=1u l=180n
CT889 t889 0 0.1f
M2247 t889 ni1 vdd vdd pch w=2u l=180n
M2248 nw235 nq69 t889 vdd pch w=2u l=180n
Cnw235 nw235 0 2f
CT890 t890 0 0.1f
M2249 t890 ni5 vdd vdd pch w=2u l=180n
M2250 t890 ni1 vdd vdd pch w=2u l=180n
CT891 t891 0 0.1f
M2251 t890 ni5 t891 0 nch w=1u l=180n
M2252 t891 ni1 0 0 nch w=1u l=180n
M2253 nw236 t890 vdd vdd pch w=2u l=180n
M2254 nw236 t890 0 0 nch w=1u l=180n
Cnw236 nw236 0 2f
CT892 t892 0 0.1f
M2255 t892 ni9 0 0 nch w=1u l=180n
M2256 t892 ni7 0 0 nch w=1u l=180n
CT893 t893 0 0.1f
M2257 t893 ni9 vdd vdd pch w=2u l=180n
M2258 t892 ni7 t893 vdd pch w=2u l=180n
M2259 nw237 t892 vdd vdd pch w=2u l=180n
M2260 nw237 t892 0 0 nch w=1u l=180n
Cnw237 nw237 0 2f
CT894 t894 0 0.1f
CT895 t895 0 0.1f
CT896 t896 0 0.1f
M2261 t894 ni13 vdd vdd pch w=2u l=180n
M2262 t894 ni14 vdd vdd pch w=2u l=180n
CT897 t897 0 0.1f
M2263 t894 ni13 t897 0 nch w=1u l=180n
M2264 t897 ni14 0 0 nch w=1u l=180n
M2265 t895 ni13 vdd vdd pch w=2u l=180n
M2266 t895 t894 vdd vdd pch w=2u l=180n
CT898 t898 0 0.1f
M2267 t895 ni13 t898 0 nch w=1u l=180n
M2268 t898 t894 0 0 nch w=1u l=180n
M2269 t896 ni14 vdd vdd pch w=2u l=180n
M2270 t896 t894 vdd vdd pch w=2u l=180n
CT899 t899 0 0.1f
M2271 t896 ni14 t899 0 nch w=1u l=180n
M2272 t899 t894 0 0 nch w=1u l=180n
M2273 nw238 t895 vdd vdd pch w=2u l=180n
M2274 nw238 t896 vdd vdd pch w=2u l=180n
CT900 t900 0 0.1f
M2275 nw238 t895 t900 0 nch w=1u l=180n
M2276 t900 t896 0 0 nch w=1u l=180n
Cnw238 nw238 0 2f
M2277 nw239 nw150 vdd vdd pch w=2u l=180n
M2278 nw239 nw152 vdd vdd pch w=2u l=180n
CT901 t901 0 0.1f
M2279 nw239 nw150 t901 0 nch w=1u l=180n
M2280 t901 nw152 0 0 nch w=1u l=180n
Cnw239 nw239 0 2f
M2281 nw240 nw154 0 0 nch w=1u l=180n
M2282 nw240 nw158 0 0 nch w=1u l=180n
CT902 t902 0 0.1f
M2283 t902 nw154 vdd vdd pch w=2u l=180n
M2284 nw240 nw158 t902 vdd pch w=2u l=180n
Cnw240 nw240 0 2f
CT903 t903 0 0.1f
M2285 t903 nw158 vdd vdd pch w=2u l=180n
M2286 t903 nw164 vdd vdd pch w=2u l=180n
CT904 t904 0 0.1f
M2287 t903 nw158 t904 0 nch w=1u l=180n
M2288 t904 nw164 0 0 nch w=1u l=180n
M2289 nw241 t903 vdd vdd pch w=2u l=180n
M2290 nw241 t903 0 0 nch w=1u l=180n
Cnw241 nw241 0 2f
CT905 t905 0 0.1f
M2291 t905 nw162 0 0 nch w=1u l=180n
M2292 t905 nw170 0 0 nch w=1u l=180n
CT906 t906 0 0.1f
M2293 t906 nw162 vdd vdd pch w=2u l=180n
M2294 t905 nw170 t906 vdd pch w=2u l=180n
M2295 nw242 t905 vdd vdd pch w=2u l=180n
M2296 nw242 t905 0 0 nch w=1u l=180n
Cnw242 nw242 0 2f
CT907 t907 0 0.1f
CT908 t908 0 0.1f
CT909 t909 0 0.1f
M2297 t907 nw166 vdd vdd pch w=2u l=180n
M2298 t907 nw176 vdd vdd pch w=2u l=180n
CT910 t910 0 0.1f
M2299 t907 nw166 t910 0 nch w=1u l=180n
M2300 t910 nw176 0 0 nch w=1u l=180n
M2301 t908 nw166 vdd vdd pch w=2u l=180n
M2302 t908 t907 vdd vdd pch w=2u l=180n
CT911 t911 0 0.1f
M2303 t908 nw166 t911 0 nch w=1u l=180n
M2304 t911 t907 0 0 nch w=1u l=180n
M2305 t909 nw176 vdd vdd pch w=2u l=180n
M2306 t909 t907 vdd vdd pch w=2u l=180n
CT912 t912 0 0.1f
M2307 t909 nw176 t912 0 nch w=1u l=180n
M2308 t912 t907 0 0 nch w=1u l=180n
M2309 nw243 t908 vdd vdd pch w=2u l=180n
M2310 nw243 t909 vdd vdd pch w=2u l=180n
CT913 t913 0 0.1f
M2311 nw243 t908 t913 0 nch w=1u l=180n
M2312 t913 t909 0 0 nch w=1u l=180n
Cnw243 nw243 0 2f
M2313 nw244 nw170 vdd vdd pch w=2u l=180n
M2314 nw244 nw182 vdd vdd pch w=2u l=180n
CT914 t914 0 0.1f
M2315 nw244 nw170 t914 0 nch w=1u l=180n
M2316 t914 nw182 0 0 nch w=1u l=180n
Cnw244 nw244 0 2f
M2317 nw245 nw174 0 0 nch w=1u l=180n
M2318 nw245 nw188 0 0 nch w=1u l=180n
CT915 t915 0 0.1f
M2319 t915 nw174 vdd vdd pch w=2u l=180n
M2320 nw245 nw188 t915 vdd pch w=2u l=180n
Cnw245 nw245 0 2f
CT916 t916 0 0.1f
M2321 t916 nw178 vdd vdd pch w=2u l=180n
M2322 t916 nw194 vdd vdd pch w=2u l=180n
CT917 t917 0 0.1f
M2323 t916 nw178 t917 0 nch w=1u l=180n
M2324 t917 nw194 0 0 nch w=1u l=180n
M2325 nw246 t916 vdd vdd pch w=2u l=180n
M2326 nw246 t916 0 0 nch w=1u l=180n
Cnw246 nw246 0 2f
CT918 t918 0 0.1f
M2327 t918 nw182 0 0 nch w=1u l=180n
M2328 t918 nw200 0 0 nch w=1u l=180n
CT919 t919 0 0.1f
M2329 t919 nw182 vdd vdd pch w=2u l=180n
M2330 t918 nw200 t919 vdd pch w=2u l=180n
M2331 nw247 t918 vdd vdd pch w=2u l=180n
M2332 nw247 t918 0 0 nch w=1u l=180n
Cnw247 nw247 0 2f
CT920 t920 0 0.1f
CT921 t921 0 0.1f
CT922 t922 0 0.1f
M2333 t920 nw186 vdd vdd pch w=2u l=180n
M2334 t920 nw206 vdd vdd pch w=2u l=180n
CT923 t923 0 0.1f
M2335 t920 nw186 t923 0 nch w=1u l=180n
M2336 t923 nw206 0 0 nch w=1u l=180n
M2337 t921 nw186 vdd vdd pch w=2u l=180n
M2338 t921 t920 vdd vdd pch w=2u l=180n
CT924 t924 0 0.1f
M2339 t921 nw186 t924 0 nch w=1u l=180n
M2340 t924 t920 0 0 nch w=1u l=180n
M2341 t922 nw206 vdd vdd pch w=2u l=180n
M2342 t922 t920 vdd vdd pch w=2u l=180n
CT925 t925 0 0.1f
M2343 t922 nw206 t925 0 nch w=1u l=180n
M2344 t925 t920 0 0 nch w=1u l=180n
M2345 nw248 t921 vdd vdd pch w=2u l=180n
M2346 nw248 t922 vdd vdd pch w=2u l=180n
CT926 t926 0 0.1f
M2347 nw248 t921 t926 0 nch w=1u l=180n
M2348 t926 t922 0 0 nch w=1u l=180n
Cnw248 nw248 0 2f
M2349 nw249 nw190 vdd vdd pch w=2u l=180n
M2350 nw249 nw212 vdd vdd pch w=2u l=180n
CT927 t927 0 0.1f
M2351 nw249 nw190 t927 0 nch w=1u l=180n
M2352 t927 nw212 0 0 nch w=1u l=180n
Cnw249 nw249 0 2f
M2353 nw250 nw194 0 0 nch w=1u l=180n
M2354 nw250 nw218 0 0 nch w=1u l=180n
CT928 t928 0 0.1f
M2355 t928 nw194 vdd vdd pch w=2u l=180n
M2356 nw250 nw218 t928 vdd pch w=2u l=180n
Cnw250 nw250 0 2f
CT929 t929 0 0.1f
M2357 t929 nw198 vdd vdd pch w=2u l=180n
M2358 t929 nw224 vdd vdd pch w=2u l=180n
CT930 t930 0 0.1f
M2359 t929 nw198 t930 0 nch w=1u l=180n
M2360 t930 nw224 0 0 nch w=1u l=180n
M2361 nw251 t929 vdd vdd pch w=2u l=180n
M2362 nw251 t929 0 0 nch w=1u l=180n
Cnw251 nw251 0 2f
CT931 t931 0 0.1f
M2363 t931 nw202 0 0 nch w=1u l=180n
M2364 t931 nw230 0 0 nch w=1u l=180n
CT932 t932 0 0.1f
M2365 t932 nw202 vdd vdd pch w=2u l=180n
M2366 t931 nw230 t932 vdd pch w=2u l=180n
M2367 nw252 t931 vdd vdd pch w=2u l=180n
M2368 nw252 t931 0 0 nch w=1u l=180n
Cnw252 nw252 0 2f
CT933 t933 0 0.1f
CT934 t934 0 0.1f
CT935 t935 0 0.1f
M2369 t933 nw206 vdd vdd pch w=2u l=180n
M2370 t933 nw236 vdd vdd pch w=2u l=180n
CT936 t936 0 0.1f
M2371 t933 nw206 t936 0 nch w=1u l=180n
M2372 t936 nw236 0 0 nch w=1u l=180n
M2373 t934 nw206 vdd vdd pch w=2u l=180n
M2374 t934 t933 vdd vdd pch w=2u l=180n
CT937 t937 0 0.1f
M2375 t934 nw206 t937 0 nch w=1u l=180n
M2376 t937 t933 0 0 nch w=1u l=180n
M2377 t935 nw236 vdd vdd pch w=2u l=180n
M2378 t935 t933 vdd vdd pch w=2u l=180n
CT938 t938 0 0.1f
M2379 t935 nw236 t938 0 nch w=1u l=180n
M2380 t938 t933 0 0 nch w=1u l=180n
M2381 nw253 t934 vdd vdd pch w=2u l=180n
M2382 nw253 t935 vdd vdd pch w=2u l=180n
CT939 t939 0 0.1f
M2383 nw253 t934 t939 0 nch w=1u l=180n
M2384 t939 t935 0 0 nch w=1u l=180n
Cnw253 nw253 0 2f
M2385 nw254 nw210 vdd vdd pch w=2u l=180n
M2386 nw254 nw242 vdd vdd pch w=2u l=180n
CT940 t940 0 0.1f
M2387 nw254 nw210 t940 0 nch w=1u l=180n
M2388 t940 nw242 0 0 nch w=1u l=180n
Cnw254 nw254 0 2f
M2389 nw255 nw214 0 0 nch w=1u l=180n
M2390 nw255 nw248 0 0 nch w=1u l=180n
CT941 t941 0 0.1f
M2391 t941 nw214 vdd vdd pch w=2u l=180n
M2392 nw255 nw248 t941 vdd pch w=2u l=180n
Cnw255 nw255 0 2f
CT942 t942 0 0.1f
M2393 t942 nw218 vdd vdd pch w=2u l=180n
M2394 t942 nw254 vdd vdd pch w=2u l=180n
CT943 t943 0 0.1f
M2395 t942 nw218 t943 0 nch w=1u l=180n
M2396 t943 nw254 0 0 nch w=1u l=180n
M2397 nw256 t942 vdd vdd pch w=2u l=180n
M2398 nw256 t942 0 0 nch w=1u l=180n
Cnw256 nw256 0 2f
CT944 t944 0 0.1f
M2399 t944 nw222 0 0 nch w=1u l=180n
M2400 t944 nq3 0 0 nch w=1u l=180n
CT945 t945 0 0.1f
M2401 t945 nw222 vdd vdd pch w=2u l=180n
M2402 t944 nq3 t945 vdd pch w=2u l=180n
M2403 nw257 t944 vdd vdd pch w=2u l=180n
M2404 nw257 t944 0 0 nch w=1u l=180n
Cnw257 nw257 0 2f
CT946 t946 0 0.1f
CT947 t947 0 0.1f
CT948 t948 0 0.1f
M2405 t946 nw226 vdd vdd pch w=2u l=180n
M2406 t946 nq8 vdd vdd pch w=2u l=180n
CT949 t949 0 0.1f
M2407 t946 nw226 t949 0 nch w=1u l=180n
M2408 t949 nq8 0 0 nch w=1u l=180n
M2409 t947 nw226 vdd vdd pch w=2u l=180n
M2410 t947 t946 vdd vdd pch w=2u l=180n
CT950 t950 0 0.1f
M2411 t947 nw226 t950 0 nch w=1u l=180n
M2412 t950 t946 0 0 nch w=1u l=180n
M2413 t948 nq8 vdd vdd pch w=2u l=180n
M2414 t948 t946 vdd vdd pch w=2u l=180n
CT951 t951 0 0.1f
M2415 t948 nq8 t951 0 nch w=1u l=180n
M2416 t951 t946 0 0 nch w=1u l=180n
M2417 nw258 t947 vdd vdd pch w=2u l=180n
M2418 nw258 t948 vdd vdd pch w=2u l=180n
CT952 t952 0 0.1f
M2419 nw258 t947 t952 0 nch w=1u l=180n
M2420 t952 t948 0 0 nch w=1u l=180n
Cnw258 nw258 0 2f
M2421 nw259 nw230 vdd vdd pch w=2u l=180n
M2422 nw259 nq13 vdd vdd pch w=2u l=180n
CT953 t953 0 0.1f
M2423 nw259 nw230 t953 0 nch w=1u l=180n
M2424 t953 nq13 0 0 nch w=1u l=180n
Cnw259 nw259 0 2f
M2425 nw260 nw234 0 0 nch w=1u l=180n
M2426 nw260 nq18 0 0 nch w=1u l=180n
CT954 t954 0 0.1f
M2427 t954 nw234 vdd vdd pch w=2u l=180n
M2428 nw260 nq18 t954 vdd pch w=2u l=180n
Cnw260 nw260 0 2f
CT955 t955 0 0.1f
M2429 t955 nw238 vdd vdd pch w=2u l=180n
M2430 t955 nq23 vdd vdd pch w=2u l=180n
CT956 t956 0 0.1f
M2431 t955 nw238 t956 0 nch w=1u l=180n
M2432 t956 nq23 0 0 nch w=1u l=180n
M2433 nw261 t955 vdd vdd pch w=2u l=180n
M2434 nw261 t955 0 0 nch w=1u l=180n
Cnw261 nw261 0 2f
CT957 t957 0 0.1f
M2435 t957 nw242 0 0 nch w=1u l=180n
M2436 t957 nq28 0 0 nch w=1u l=180n
CT958 t958 0 0.1f
M2437 t958 nw242 vdd vdd pch w=2u l=180n
M2438 t957 nq28 t958 vdd pch w=2u l=180n
M2439 nw262 t957 vdd vdd pch w=2u l=180n
M2440 nw262 t957 0 0 nch w=1u l=180n
Cnw262 nw262 0 2f
CT959 t959 0 0.1f
CT960 t960 0 0.1f
CT961 t961 0 0.1f
M2441 t959 nw246 vdd vdd pch w=2u l=180n
M2442 t959 nq33 vdd vdd pch w=2u l=180n
CT962 t962 0 0.1f
M2443 t959 nw246 t962 0 nch w=1u l=180n
M2444 t962 nq33 0 0 nch w=1u l=180n
M2445 t960 nw246 vdd vdd pch w=2u l=180n
M2446 t960 t959 vdd vdd pch w=2u l=180n
CT963 t963 0 0.1f
M2447 t960 nw246 t963 0 nch w=1u l=180n
M2448 t963 t959 0 0 nch w=1u l=180n
M2449 t961 nq33 vdd vdd pch w=2u l=180n
M2450 t961 t959 vdd vdd pch w=2u l=180n
CT964 t964 0 0.1f
M2451 t961 nq33 t964 0 nch w=1u l=180n
M2452 t964 t959 0 0 nch w=1u l=180n
M2453 nw263 t960 vdd vdd pch w=2u l=180n
M2454 nw263 t961 vdd vdd pch w=2u l=180n
CT965 t965 0 0.1f
M2455 nw263 t960 t965 0 nch w=1u l=180n
M2456 t965 t961 0 0 nch w=1u l=180n
Cnw263 nw263 0 2f
M2457 nw264 nw250 vdd vdd pch w=2u l=180n
M2458 nw264 nq38 vdd vdd pch w=2u l=180n
CT966 t966 0 0.1f
M2459 nw264 nw250 t966 0 nch w=1u l=180n
M2460 t966 nq38 0 0 nch w=1u l=180n
Cnw264 nw264 0 2f
M2461 nw265 nw254 0 0 nch w=1u l=180n
M2462 nw265 nq43 0 0 nch w=1u l=180n
CT967 t967 0 0.1f
M2463 t967 nw254 vdd vdd pch w=2u l=180n
M2464 nw265 nq43 t967 vdd pch w=2u l=180n
Cnw265 nw265 0 2f
CT968 t968 0 0.1f
M2465 t968 nw258 vdd vdd pch w=2u l=180n
M2466 t968 nq48 vdd vdd pch w=2u l=180n
CT969 t969 0 0.1f
M2467 t968 nw258 t969 0 nch w=1u l=180n
M2468 t969 nq48 0 0 nch w=1u l=180n
M2469 nw266 t968 vdd vdd pch w=2u l=180n
M2470 nw266 t968 0 0 nch w=1u l=180n
Cnw266 nw266 0 2f
CT970 t970 0 0.1f
M2471 t970 nw262 0 0 nch w=1u l=180n
M2472 t970 nq53 0 0 nch w=1u l=180n
CT971 t971 0 0.1f
M2473 t971 nw262 vdd vdd pch w=2u l=180n
M2474 t970 nq53 t971 vdd pch w=2u l=180n
M2475 nw267 t970 vdd vdd pch w=2u l=180n
M2476 nw267 t970 0 0 nch w=1u l=180n
Cnw267 nw267 0 2f
CT972 t972 0 0.1f
CT973 t973 0 0.1f
CT974 t974 0 0.1f
M2477 t972 nw266 vdd vdd pch w=2u l=180n
M2478 t972 nq58 vdd vdd pch w=2u l=180n
CT975 t975 0 0.1f
M2479 t972 nw266 t975 0 nch w=1u l=180n
M2480 t975 nq58 0 0 nch w=1u l=180n
M2481 t973 nw266 vdd vdd pch w=2u l=180n
M2482 t973 t972 vdd vdd pch w=2u l=180n
CT976 t976 0 0.1f
M2483 t973 nw266 t976 0 nch w=1u l=180n
M2484 t976 t972 0 0 nch w=1u l=180n
M2485 t974 nq58 vdd vdd pch w=2u l=180n
M2486 t974 t972 vdd vdd pch w=2u l=180n
CT977 t977 0 0.1f
M2487 t974 nq58 t977 0 nch w=1u l=180n
M2488 t977 t972 0 0 nch w=1u l=180n
M2489 nw268 t973 vdd vdd pch w=2u l=180n
M2490 nw268 t974 vdd vdd pch w=2u l=180n
CT978 t978 0 0.1f
M2491 nw268 t973 t978 0 nch w=1u l=180n
M2492 t978 t974 0 0 nch w=1u l=180n
Cnw268 nw268 0 2f
M2493 nw269 nq1 vdd vdd pch w=2u l=180n
M2494 nw269 nq63 vdd vdd pch w=2u l=180n
CT979 t979 0 0.1f
M2495 nw269 nq1 t979 0 nch w=1u l=180n
M2496 t979 nq63 0 0 nch w=1u l=180n
Cnw269 nw269 0 2f
M2497 nw270 nq4 0 0 nch w=1u l=180n
M2498 nw270 nq68 0 0 nch w=1u l=180n
CT980 t980 0 0.1f
M2499 t980 nq4 vdd vdd pch w=2u l=180n
M2500 nw270 nq68 t980 vdd pch w=2u l=180n
Cnw270 nw270 0 2f
CT981 t981 0 0.1f
M2501 t981 nq7 vdd vdd pch w=2u l=180n
M2502 t981 nq73 vdd vdd pch w=2u l=180n
CT982 t982 0 0.1f
M2503 t981 nq7 t982 0 nch w=1u l=180n
M2504 t982 nq73 0 0 nch w=1u l=180n
M2505 nw271 t981 vdd vdd pch w=2u l=180n
M2506 nw271 t981 0 0 nch w=1u l=180n
Cnw271 nw271 0 2f
CT983 t983 0 0.1f
M2507 t983 nq10 0 0 nch w=1u l=180n
M2508 t983 ni4 0 0 nch w=1u l=180n
CT984 t984 0 0.1f
M2509 t984 nq10 vdd vdd pch w=2u l=180n
M2510 t983 ni4 t984 vdd pch w=2u l=180n
M2511 nw272 t983 vdd vdd pch w=2u l=180n
M2512 nw272 t983 0 0 nch w=1u l=180n
Cnw272 nw272 0 2f
CT985 t985 0 0.1f
CT986 t986 0 0.1f
CT987 t987 0 0.1f
M2513 t985 nq13 vdd vdd pch w=2u l=180n
M2514 t985 ni9 vdd vdd pch w=2u l=180n
CT988 t988 0 0.1f
M2515 t985 nq13 t988 0 nch w=1u l=180n
M2516 t988 ni9 0 0 nch w=1u l=180n
M2517 t986 nq13 vdd vdd pch w=2u l=180n
M2518 t986 t985 vdd vdd pch w=2u l=180n
CT989 t989 0 0.1f
M2519 t986 nq13 t989 0 nch w=1u l=180n
M2520 t989 t985 0 0 nch w=1u l=180n
M2521 t987 ni9 vdd vdd pch w=2u l=180n
M2522 t987 t985 vdd vdd pch w=2u l=180n
CT990 t990 0 0.1f
M2523 t987 ni9 t990 0 nch w=1u l=180n
M2524 t990 t985 0 0 nch w=1u l=180n
M2525 nw273 t986 vdd vdd pch w=2u l=180n
M2526 nw273 t987 vdd vdd pch w=2u l=180n
CT991 t991 0 0.1f
M2527 nw273 t986 t991 0 nch w=1u l=180n
M2528 t991 t987 0 0 nch w=1u l=180n
Cnw273 nw273 0 2f
M2529 nw274 nq16 vdd vdd pch w=2u l=180n
M2530 nw274 ni14 vdd vdd pch w=2u l=180n
CT992 t992 0 0.1f
M2531 nw274 nq16 t992 0 nch w=1u l=180n
M2532 t992 ni14 0 0 nch w=1u l=180n
Cnw274 nw274 0 2f
M2533 nw275 nq19 0 0 nch w=1u l=180n
M2534 nw275 nw152 0 0 nch w=1u l=180n
CT993 t993 0 0.1f
M2535 t993 nq19 vdd vdd pch w=2u l=180n
M2536 nw275 nw152 t993 vdd pch w=2u l=180n
Cnw275 nw275 0 2f
CT994 t994 0 0.1f
M2537 t994 nq22 vdd vdd pch w=2u l=180n
M2538 t994 nw157 vdd vdd pch w=2u l=180n
CT995 t995 0 0.1f
M2539 t994 nq22 t995 0 nch w=1u l=180n
M2540 t995 nw157 0 0 nch w=1u l=180n
M2541 nw276 t994 vdd vdd pch w=2u l=180n
M2542 nw276 t994 0 0 nch w=1u l=180n
Cnw276 nw276 0 2f
CT996 t996 0 0.1f
M2543 t996 nq25 0 0 nch w=1u l=180n
M2544 t996 nw162 0 0 nch w=1u l=180n
CT997 t997 0 0.1f
M2545 t997 nq25 vdd vdd pch w=2u l=180n
M2546 t996 nw162 t997 vdd pch w=2u l=180n
M2547 nw277 t996 vdd vdd pch w=2u l=180n
M2548 nw277 t996 0 0 nch w=1u l=180n
Cnw277 nw277 0 2f
CT998 t998 0 0.1f
CT999 t999 0 0.1f
CT1000 t1000 0 0.1f
M2549 t998 nq28 vdd vdd pch w=2u l=180n
M2550 t998 nw167 vdd vdd pch w=2u l=180n
CT1001 t1001 0 0.1f
M2551 t998 nq28 t1001 0 nch w=1u l=180n
M2552 t1001 nw167 0 0 nch w=1u l=180n
M2553 t999 nq28 vdd vdd pch w=2u l=180n
M2554 t999 t998 vdd vdd pch w=2u l=180n
CT1002 t1002 0 0.1f
M2555 t999 nq28 t1002 0 nch w=1u l=180n
M2556 t1002 t998 0 0 nch w=1u l=180n
M2557 t1000 nw167 vdd vdd pch w=2u l=180n
M2558 t1000 t998 vdd vdd pch w=2u l=180n
CT1003 t1003 0 0.1f
M2559 t1000 nw167 t1003 0 nch w=1u l=180n
M2560 t1003 t998 0 0 nch w=1u l=180n
M2561 nw278 t999 vdd vdd pch w=2u l=180n
M2562 nw278 t1000 vdd vdd pch w=2u l=180n
CT1004 t1004 0 0.1f
M2563 nw278 t999 t1004 0 nch w=1u l=180n
M2564 t1004 t1000 0 0 nch w=1u l=180n
Cnw278 nw278 0 2f
M2565 nw279 nq31 vdd vdd pch w=2u l=180n
M2566 nw279 nw172 vdd vdd pch w=2u l=180n
CT1005 t1005 0 0.1f
M2567 nw279 nq31 t1005 0 nch w=1u l=180n
M2568 t1005 nw172 0 0 nch w=1u l=180n
Cnw279 nw279 0 2f
M2569 nw280 nq34 0 0 nch w=1u l=180n
M2570 nw280 nw177 0 0 nch w=1u l=180n
CT1006 t1006 0 0.1f
M2571 t1006 nq34 vdd vdd pch w=2u l=180n
M2572 nw280 nw177 t1006 vdd pch w=2u l=180n
Cnw280 nw280 0 2f
CT1007 t1007 0 0.1f
M2573 t1007 nq37 vdd vdd pch w=2u l=180n
M2574 t1007 nw182 vdd vdd pch w=2u l=180n
CT1008 t1008 0 0.1f
M2575 t1007 nq37 t1008 0 nch w=1u l=180n
M2576 t1008 nw182 0 0 nch w=1u l=180n
M2577 nw281 t1007 vdd vdd pch w=2u l=180n
M2578 nw281 t1007 0 0 nch w=1u l=180n
Cnw281 nw281 0 2f
CT1009 t1009 0 0.1f
M2579 t1009 nq40 0 0 nch w=1u l=180n
M2580 t1009 nw187 0 0 nch w=1u l=180n
CT1010 t1010 0 0.1f
M2581 t1010 nq40 vdd vdd pch w=2u l=180n
M2582 t1009 nw187 t1010 vdd pch w=2u l=180n
M2583 nw282 t1009 vdd vdd pch w=2u l=180n
M2584 nw282 t1009 0 0 nch w=1u l=180n
Cnw282 nw282 0 2f
CT1011 t1011 0 0.1f
CT1012 t1012 0 0.1f
CT1013 t1013 0 0.1f
M2585 t1011 nq43 vdd vdd pch w=2u l=180n
M2586 t1011 nw192 vdd vdd pch w=2u l=180n
CT1014 t1014 0 0.1f
M2587 t1011 nq43 t1014 0 nch w=1u l=180n
M2588 t1014 nw192 0 0 nch w=1u l=180n
M2589 t1012 nq43 vdd vdd pch w=2u l=180n
M2590 t1012 t1011 vdd vdd pch w=2u l=180n
CT1015 t1015 0 0.1f
M2591 t1012 nq43 t1015 0 nch w=1u l=180n
M2592 t1015 t1011 0 0 nch w=1u l=180n
M2593 t1013 nw192 vdd vdd pch w=2u l=180n
M2594 t1013 t1011 vdd vdd pch w=2u l=180n
CT1016 t1016 0 0.1f
M2595 t1013 nw192 t1016 0 nch w=1u l=180n
M2596 t1016 t1011 0 0 nch w=1u l=180n
M2597 nw283 t1012 vdd vdd pch w=2u l=180n
M2598 nw283 t1013 vdd vdd pch w=2u l=180n
CT1017 t1017 0 0.1f
M2599 nw283 t1012 t1017 0 nch w=1u l=180n
M2600 t1017 t1013 0 0 nch w=1u l=180n
Cnw283 nw283 0 2f
M2601 nw284 nq46 vdd vdd pch w=2u l=180n
M2602 nw284 nw197 vdd vdd pch w=2u l=180n
CT1018 t1018 0 0.1f
M2603 nw284 nq46 t1018 0 nch w=1u l=180n
M2604 t1018 nw197 0 0 nch w=1u l=180n
Cnw284 nw284 0 2f
M2605 nw285 nq49 0 0 nch w=1u l=180n
M2606 nw285 nw202 0 0 nch w=1u l=180n
CT1019 t1019 0 0.1f
M2607 t1019 nq49 vdd vdd pch w=2u l=180n
M2608 nw285 nw202 t1019 vdd pch w=2u l=180n
Cnw285 nw285 0 2f
CT1020 t1020 0 0.1f
M2609 t1020 nq52 vdd vdd pch w=2u l=180n
M2610 t1020 nw207 vdd vdd pch w=2u l=180n
CT1021 t1021 0 0.1f
M2611 t1020 nq52 t1021 0 nch w=1u l=180n
M2612 t1021 nw207 0 0 nch w=1u l=180n
M2613 nw286 t1020 vdd vdd pch w=2u l=180n
M2614 nw286 t1020 0 0 nch w=1u l=180n
Cnw286 nw286 0 2f
CT1022 t1022 0 0.1f
M2615 t1022 nq55 0 0 nch w=1u l=180n
M2616 t1022 nw212 0 0 nch w=1u l=180n
CT1023 t1023 0 0.1f
M2617 t1023 nq55 vdd vdd pch w=2u l=180n
M2618 t1022 nw212 t1023 vdd pch w=2u l=180n
M2619 nw287 t1022 vdd vdd pch w=2u l=180n
M2620 nw287 t1022 0 0 nch w=1u l=180n
Cnw287 nw287 0 2f
CT1024 t1024 0 0.1f
CT1025 t1025 0 0.1f
CT1026 t1026 0 0.1f
M2621 t1024 nq58 vdd vdd pch w=2u l=180n
M2622 t1024 nw217 vdd vdd pch w=2u l=180n
CT1027 t1027 0 0.1f
M2623 t1024 nq58 t1027 0 nch w=1u l=180n
M2624 t1027 nw217 0 0 nch w=1u l=180n
M2625 t1025 nq58 vdd vdd pch w=2u l=180n
M2626 t1025 t1024 vdd vdd pch w=2u l=180n
CT1028 t1028 0 0.1f
M2627 t1025 nq58 t1028 0 nch w=1u l=180n
M2628 t1028 t1024 0 0 nch w=1u l=180n
M2629 t1026 nw217 vdd vdd pch w=2u l=180n
M2630 t1026 t1024 vdd vdd pch w=2u l=180n
CT1029 t1029 0 0.1f
M2631 t1026 nw217 t1029 0 nch w=1u l=180n
M2632 t1029 t1024 0 0 nch w=1u l=180n
M2633 nw288 t1025 vdd vdd pch w=2u l=180n
M2634 nw288 t1026 vdd vdd pch w=2u l=180n
CT1030 t1030 0 0.1f
M2635 nw288 t1025 t1030 0 nch w=1u l=180n
M2636 t1030 t1026 0 0 nch w=1u l=180n
Cnw288 nw288 0 2f
M2637 nw289 nq61 vdd vdd pch w=2u l=180n
M2638 nw289 nw222 vdd vdd pch w=2u l=180n
CT1031 t1031 0 0.1f
M2639 nw289 nq61 t1031 0 nch w=1u l=180n
M2640 t1031 nw222 0 0 nch w=1u l=180n
Cnw289 nw289 0 2f
M2641 nw290 nq64 0 0 nch w=1u l=180n
M2642 nw290 nw227 0 0 nch w=1u l=180n
CT1032 t1032 0 0.1f
M2643 t1032 nq64 vdd vdd pch w=2u l=180n
M2644 nw290 nw227 t1032 vdd pch w=2u l=180n
Cnw290 nw290 0 2f
CT1033 t1033 0 0.1f
M2645 t1033 nq67 vdd vdd pch w=2u l=180n
M2646 t1033 nw232 vdd vdd pch w=2u l=180n
CT1034 t1034 0 0.1f
M2647 t1033 nq67 t1034 0 nch w=1u l=180n
M2648 t1034 nw232 0 0 nch w=1u l=180n
M2649 nw291 t1033 vdd vdd pch w=2u l=180n
M2650 nw291 t1033 0 0 nch w=1u l=180n
Cnw291 nw291 0 2f
CT1035 t1035 0 0.1f
M2651 t1035 nq70 0 0 nch w=1u l=180n
M2652 t1035 nw237 0 0 nch w=1u l=180n
CT1036 t1036 0 0.1f
M2653 t1036 nq70 vdd vdd pch w=2u l=180n
M2654 t1035 nw237 t1036 vdd pch w=2u l=180n
M2655 nw292 t1035 vdd vdd pch w=2u l=180n
M2656 nw292 t1035 0 0 nch w=1u l=180n
Cnw292 nw292 0 2f
CT1037 t1037 0 0.1f
CT1038 t1038 0 0.1f
CT1039 t1039 0 0.1f
M2657 t1037 nq73 vdd vdd pch w=2u l=180n
M2658 t1037 nw242 vdd vdd pch w=2u l=180n
CT1040 t1040 0 0.1f
M2659 t1037 nq73 t1040 0 nch w=1u l=180n
M2660 t1040 nw242 0 0 nch w=1u l=180n
M2661 t1038 nq73 vdd vdd pch w=2u l=180n
M2662 t1038 t1037 vdd vdd pch w=2u l=180n
CT1041 t1041 0 0.1f
M2663 t1038 nq73 t1041 0 nch w=1u l=180n
M2664 t1041 t1037 0 0 nch w=1u l=180n
M2665 t1039 nw242 vdd vdd pch w=2u l=180n
M2666 t1039 t1037 vdd vdd pch w=2u l=180n
CT1042 t1042 0 0.1f
M2667 t1039 nw242 t1042 0 nch w=1u l=180n
M2668 t1042 t1037 0 0 nch w=1u l=180n
M2669 nw293 t1038 vdd vdd pch w=2u l=180n
M2670 nw293 t1039 vdd vdd pch w=2u l=180n
CT1043 t1043 0 0.1f
M2671 nw293 t1038 t1043 0 nch w=1u l=180n
M2672 t1043 t1039 0 0 nch w=1u l=180n
Cnw293 nw293 0 2f
M2673 nw294 ni2 vdd vdd pch w=2u l=180n
M2674 nw294 nw247 vdd vdd pch w=2u l=180n
CT1044 t1044 0 0.1f
M2675 nw294 ni2 t1044 0 nch w=1u l=180n
M2676 t1044 nw247 0 0 nch w=1u l=180n
Cnw294 nw294 0 2f
M2677 nw295 ni5 0 0 nch w=1u l=180n
M2678 nw295 nw252 0 0 nch w=1u l=180n
CT1045 t1045 0 0.1f
M2679 t1045 ni5 vdd vdd pch w=2u l=180n
M2680 nw295 nw252 t1045 vdd pch w=2u l=180n
Cnw295 nw295 0 2f
CT1046 t1046 0 0.1f
M2681 t1046 ni8 vdd vdd pch w=2u l=180n
M2682 t1046 nw257 vdd vdd pch w=2u l=180n
CT1047 t1047 0 0.1f
M2683 t1046 ni8 t1047 0 nch w=1u l=180n
M2684 t1047 nw257 0 0 nch w=1u l=180n
M2685 nw296 t1046 vdd vdd pch w=2u l=180n
M2686 nw296 t1046 0 0 nch w=1u l=180n
Cnw296 nw296 0 2f
CT1048 t1048 0 0.1f
M2687 t1048 ni11 0 0 nch w=1u l=180n
M2688 t1048 nw262 0 0 nch w=1u l=180n
CT1049 t1049 0 0.1f
M2689 t1049 ni11 vdd vdd pch w=2u l=180n
M2690 t1048 nw262 t1049 vdd pch w=2u l=180n
M2691 nw297 t1048 vdd vdd pch w=2u l=180n
M2692 nw297 t1048 0 0 nch w=1u l=180n
Cnw297 nw297 0 2f
CT1050 t1050 0 0.1f
CT1051 t1051 0 0.1f
CT1052 t1052 0 0.1f
M2693 t1050 ni14 vdd vdd pch w=2u l=180n
M2694 t1050 nw267 vdd vdd pch w=2u l=180n
CT1053 t1053 0 0.1f
M2695 t1050 ni14 t1053 0 nch w=1u l=180n
M2696 t1053 nw267 0 0 nch w=1u l=180n
M2697 t1051 ni14 vdd vdd pch w=2u l=180n
M2698 t1051 t1050 vdd vdd pch w=2u l=180n
CT1054 t1054 0 0.1f
M2699 t1051 ni14 t1054 0 nch w=1u l=180n
M2700 t1054 t1050 0 0 nch w=1u l=180n
M2701 t1052 nw267 vdd vdd pch w=2u l=180n
M2702 t1052 t1050 vdd vdd pch w=2u l=180n
CT1055 t1055 0 0.1f
M2703 t1052 nw267 t1055 0 nch w=1u l=180n
M2704 t1055 t1050 0 0 nch w=1u l=180n
M2705 nw298 t1051 vdd vdd pch w=2u l=180n
M2706 nw298 t1052 vdd vdd pch w=2u l=180n
CT1056 t1056 0 0.1f
M2707 nw298 t1051 t1056 0 nch w=1u l=180n
M2708 t1056 t1052 0 0 nch w=1u l=180n
Cnw298 nw298 0 2f
M2709 nw299 nw150 vdd vdd pch w=2u l=180n
M2710 nw299 nw272 vdd vdd pch w=2u l=180n
CT1057 t1057 0 0.1f
M2711 nw299 nw150 t1057 0 nch w=1u l=180n
M2712 t1057 nw272 0 0 nch w=1u l=180n
Cnw299 nw299 0 2f
M2713 nw300 nw153 0 0 nch w=1u l=180n
M2714 nw300 nw277 0 0 nch w=1u l=180n
CT1058 t1058 0 0.1f
M2715 t1058 nw153 vdd vdd pch w=2u l=180n
M2716 nw300 nw277 t1058 vdd pch w=2u l=180n
Cnw300 nw300 0 2f
CT1059 t1059 0 0.1f
M2717 t1059 nw156 vdd vdd pch w=2u l=180n
M2718 t1059 nw282 vdd vdd pch w=2u l=180n
CT1060 t1060 0 0.1f
M2719 t1059 nw156 t1060 0 nch w=1u l=180n
M2720 t1060 nw282 0 0 nch w=1u l=180n
M2721 nw301 t1059 vdd vdd pch w=2u l=180n
M2722 nw301 t1059 0 0 nch w=1u l=180n
Cnw301 nw301 0 2f
CT1061 t1061 0 0.1f
M2723 t1061 nw159 0 0 nch w=1u l=180n
M2724 t1061 nw287 0 0 nch w=1u l=180n
CT1062 t1062 0 0.1f
M2725 t1062 nw159 vdd vdd pch w=2u l=180n
M2726 t1061 nw287 t1062 vdd pch w=2u l=180n
M2727 nw302 t1061 vdd vdd pch w=2u l=180n
M2728 nw302 t1061 0 0 nch w=1u l=180n
Cnw302 nw302 0 2f
CT1063 t1063 0 0.1f
CT1064 t1064 0 0.1f
CT1065 t1065 0 0.1f
M2729 t1063 nw162 vdd vdd pch w=2u l=180n
M2730 t1063 nw292 vdd vdd pch w=2u l=180n
CT1066 t1066 0 0.1f
M2731 t1063 nw162 t1066 0 nch w=1u l=180n
M2732 t1066 nw292 0 0 nch w=1u l=180n
M2733 t1064 nw162 vdd vdd pch w=2u l=180n
M2734 t1064 t1063 vdd vdd pch w=2u l=180n
CT1067 t1067 0 0.1f
M2735 t1064 nw162 t1067 0 nch w=1u l=180n
M2736 t1067 t1063 0 0 nch w=1u l=180n
M2737 t1065 nw292 vdd vdd pch w=2u l=180n
M2738 t1065 t1063 vdd vdd pch w=2u l=180n
CT1068 t1068 0 0.1f
M2739 t1065 nw292 t1068 0 nch w=1u l=180n
M2740 t1068 t1063 0 0 nch w=1u l=180n
M2741 nw303 t1064 vdd vdd pch w=2u l=180n
M2742 nw303 t1065 vdd vdd pch w=2u l=180n
CT1069 t1069 0 0.1f
M2743 nw303 t1064 t1069 0 nch w=1u l=180n
M2744 t1069 t1065 0 0 nch w=1u l=180n
Cnw303 nw303 0 2f
M2745 nw304 nw165 vdd vdd pch w=2u l=180n
M2746 nw304 nw297 vdd vdd pch w=2u l=180n
CT1070 t1070 0 0.1f
M2747 nw304 nw165 t1070 0 nch w=1u l=180n
M2748 t1070 nw297 0 0 nch w=1u l=180n
Cnw304 nw304 0 2f
M2749 nw305 nw168 0 0 nch w=1u l=180n
M2750 nw305 nw302 0 0 nch w=1u l=180n
CT1071 t1071 0 0.1f
M2751 t1071 nw168 vdd vdd pch w=2u l=180n
M2752 nw305 nw302 t1071 vdd pch w=2u l=180n
Cnw305 nw305 0 2f
CT1072 t1072 0 0.1f
M2753 t1072 nw171 vdd vdd pch w=2u l=180n
M2754 t1072 nq1 vdd vdd pch w=2u l=180n
CT1073 t1073 0 0.1f
M2755 t1072 nw171 t1073 0 nch w=1u l=180n
M2756 t1073 nq1 0 0 nch w=1u l=180n
M2757 nw306 t1072 vdd vdd pch w=2u l=180n
M2758 nw306 t1072 0 0 nch w=1u l=180n
Cnw306 nw306 0 2f
CT1074 t1074 0 0.1f
M2759 t1074 nw174 0 0 nch w=1u l=180n
M2760 t1074 nq5 0 0 nch w=1u l=180n
CT1075 t1075 0 0.1f
M2761 t1075 nw174 vdd vdd pch w=2u l=180n
M2762 t1074 nq5 t1075 vdd pch w=2u l=180n
M2763 nw307 t1074 vdd vdd pch w=2u l=180n
M2764 nw307 t1074 0 0 nch w=1u l=180n
Cnw307 nw307 0 2f
CT1076 t1076 0 0.1f
CT1077 t1077 0 0.1f
CT1078 t1078 0 0.1f
M2765 t1076 nw177 vdd vdd pch w=2u l=180n
M2766 t1076 nq9 vdd vdd pch w=2u l=180n
CT1079 t1079 0 0.1f
M2767 t1076 nw177 t1079 0 nch w=1u l=180n
M2768 t1079 nq9 0 0 nch w=1u l=180n
M2769 t1077 nw177 vdd vdd pch w=2u l=180n
M2770 t1077 t1076 vdd vdd pch w=2u l=180n
CT1080 t1080 0 0.1f
M2771 t1077 nw177 t1080 0 nch w=1u l=180n
M2772 t1080 t1076 0 0 nch w=1u l=180n
M2773 t1078 nq9 vdd vdd pch w=2u l=180n
M2774 t1078 t1076 vdd vdd pch w=2u l=180n
CT1081 t1081 0 0.1f
M2775 t1078 nq9 t1081 0 nch w=1u l=180n
M2776 t1081 t1076 0 0 nch w=1u l=180n
M2777 nw308 t1077 vdd vdd pch w=2u l=180n
M2778 nw308 t1078 vdd vdd pch w=2u l=180n
CT1082 t1082 0 0.1f
M2779 nw308 t1077 t1082 0 nch w=1u l=180n
M2780 t1082 t1078 0 0 nch w=1u l=180n
Cnw308 nw308 0 2f
M2781 nw309 nw180 vdd vdd pch w=2u l=180n
M2782 nw309 nq13 vdd vdd pch w=2u l=180n
CT1083 t1083 0 0.1f
M2783 nw309 nw180 t1083 0 nch w=1u l=180n
M2784 t1083 nq13 0 0 nch w=1u l=180n
Cnw309 nw309 0 2f
M2785 nw310 nw183 0 0 nch w=1u l=180n
M2786 nw310 nq17 0 0 nch w=1u l=180n
CT1084 t1084 0 0.1f
M2787 t1084 nw183 vdd vdd pch w=2u l=180n
M2788 nw310 nq17 t1084 vdd pch w=2u l=180n
Cnw310 nw310 0 2f
CT1085 t1085 0 0.1f
M2789 t1085 nw186 vdd vdd pch w=2u l=180n
M2790 t1085 nq21 vdd vdd pch w=2u l=180n
CT1086 t1086 0 0.1f
M2791 t1085 nw186 t1086 0 nch w=1u l=180n
M2792 t1086 nq21 0 0 nch w=1u l=180n
M2793 nw311 t1085 vdd vdd pch w=2u l=180n
M2794 nw311 t1085 0 0 nch w=1u l=180n
Cnw311 nw311 0 2f
CT1087 t1087 0 0.1f
M2795 t1087 nw189 0 0 nch w=1u l=180n
M2796 t1087 nq25 0 0 nch w=1u l=180n
CT1088 t1088 0 0.1f
M2797 t1088 nw189 vdd vdd pch w=2u l=180n
M2798 t1087 nq25 t1088 vdd pch w=2u l=180n
M2799 nw312 t1087 vdd vdd pch w=2u l=180n
M2800 nw312 t1087 0 0 nch w=1u l=180n
Cnw312 nw312 0 2f
CT1089 t1089 0 0.1f
CT1090 t1090 0 0.1f
CT1091 t1091 0 0.1f
M2801 t1089 nw192 vdd vdd pch w=2u l=180n
M2802 t1089 nq29 vdd vdd pch w=2u l=180n
CT1092 t1092 0 0.1f
M2803 t1089 nw192 t1092 0 nch w=1u l=180n
M2804 t1092 nq29 0 0 nch w=1u l=180n
M2805 t1090 nw192 vdd vdd pch w=2u l=180n
M2806 t1090 t1089 vdd vdd pch w=2u l=180n
CT1093 t1093 0 0.1f
M2807 t1090 nw192 t1093 0 nch w=1u l=180n
M2808 t1093 t1089 0 0 nch w=1u l=180n
M2809 t1091 nq29 vdd vdd pch w=2u l=180n
M2810 t1091 t1089 vdd vdd pch w=2u l=180n
CT1094 t1094 0 0.1f
M2811 t1091 nq29 t1094 0 nch w=1u l=180n
M2812 t1094 t1089 0 0 nch w=1u l=180n
M2813 nw313 t1090 vdd vdd pch w=2u l=180n
M2814 nw313 t1091 vdd vdd pch w=2u l=180n
CT1095 t1095 0 0.1f
M2815 nw313 t1090 t1095 0 nch w=1u l=180n
M2816 t1095 t1091 0 0 nch w=1u l=180n
Cnw313 nw313 0 2f
M2817 nw314 nw195 vdd vdd pch w=2u l=180n
M2818 nw314 nq33 vdd vdd pch w=2u l=180n
CT1096 t1096 0 0.1f
M2819 nw314 nw195 t1096 0 nch w=1u l=180n
M2820 t1096 nq33 0 0 nch w=1u l=180n
Cnw314 nw314 0 2f
M2821 nw315 nw198 0 0 nch w=1u l=180n
M2822 nw315 nq37 0 0 nch w=1u l=180n
CT1097 t1097 0 0.1f
M2823 t1097 nw198 vdd vdd pch w=2u l=180n
M2824 nw315 nq37 t1097 vdd pch w=2u l=180n
Cnw315 nw315 0 2f
CT1098 t1098 0 0.1f
M2825 t1098 nw201 vdd vdd pch w=2u l=180n
M2826 t1098 nq41 vdd vdd pch w=2u l=180n
CT1099 t1099 0 0.1f
M2827 t1098 nw201 t1099 0 nch w=1u l=180n
M2828 t1099 nq41 0 0 nch w=1u l=180n
M2829 nw316 t1098 vdd vdd pch w=2u l=180n
M2830 nw316 t1098 0 0 nch w=1u l=180n
Cnw316 nw316 0 2f
CT1100 t1100 0 0.1f
M2831 t1100 nw204 0 0 nch w=1u l=180n
M2832 t1100 nq45 0 0 nch w=1u l=180n
CT1101 t1101 0 0.1f
M2833 t1101 nw204 vdd vdd pch w=2u l=180n
M2834 t1100 nq45 t1101 vdd pch w=2u l=180n
M2835 nw317 t1100 vdd vdd pch w=2u l=180n
M2836 nw317 t1100 0 0 nch w=1u l=180n
Cnw317 nw317 0 2f
CT1102 t1102 0 0.1f
CT1103 t1103 0 0.1f
CT1104 t1104 0 0.1f
M2837 t1102 nw207 vdd vdd pch w=2u l=180n
M2838 t1102 nq49 vdd vdd pch w=2u l=180n
CT1105 t1105 0 0.1f
M2839 t1102 nw207 t1105 0 nch w=1u l=180n
M2840 t1105 nq49 0 0 nch w=1u l=180n
M2841 t1103 nw207 vdd vdd pch w=2u l=180n
M2842 t1103 t1102 vdd vdd pch w=2u l=180n
CT1106 t1106 0 0.1f
M2843 t1103 nw207 t1106 0 nch w=1u l=180n
M2844 t1106 t1102 0 0 nch w=1u l=180n
M2845 t1104 nq49 vdd vdd pch w=2u l=180n
M2846 t1104 t1102 vdd vdd pch w=2u l=180n
CT1107 t1107 0 0.1f
M2847 t1104 nq49 t1107 0 nch w=1u l=180n
M2848 t1107 t1102 0 0 nch w=1u l=180n
M2849 nw318 t1103 vdd vdd pch w=2u l=180n
M2850 nw318 t1104 vdd vdd pch w=2u l=180n
CT1108 t1108 0 0.1f
M2851 nw318 t1103 t1108 0 nch w=1u l=180n
M2852 t1108 t1104 0 0 nch w=1u l=180n
Cnw318 nw318 0 2f
M2853 nw319 nw210 vdd vdd pch w=2u l=180n
M2854 nw319 nq53 vdd vdd pch w=2u l=180n
CT1109 t1109 0 0.1f
M2855 nw319 nw210 t1109 0 nch w=1u l=180n
M2856 t1109 nq53 0 0 nch w=1u l=180n
Cnw319 nw319 0 2f
M2857 nw320 nw213 0 0 nch w=1u l=180n
M2858 nw320 nq57 0 0 nch w=1u l=180n
CT1110 t1110 0 0.1f
M2859 t1110 nw213 vdd vdd pch w=2u l=180n
M2860 nw320 nq57 t1110 vdd pch w=2u l=180n
Cnw320 nw320 0 2f
CT1111 t1111 0 0.1f
M2861 t1111 nw216 vdd vdd pch w=2u l=180n
M2862 t1111 nq61 vdd vdd pch w=2u l=180n
CT1112 t1112 0 0.1f
M2863 t1111 nw216 t1112 0 nch w=1u l=180n
M2864 t1112 nq61 0 0 nch w=1u l=180n
M2865 nw321 t1111 vdd vdd pch w=2u l=180n
M2866 nw321 t1111 0 0 nch w=1u l=180n
Cnw321 nw321 0 2f
CT1113 t1113 0 0.1f
M2867 t1113 nw219 0 0 nch w=1u l=180n
M2868 t1113 nq65 0 0 nch w=1u l=180n
CT1114 t1114 0 0.1f
M2869 t1114 nw219 vdd vdd pch w=2u l=180n
M2870 t1113 nq65 t1114 vdd pch w=2u l=180n
M2871 nw322 t1113 vdd vdd pch w=2u l=180n
M2872 nw322 t1113 0 0 nch w=1u l=180n
Cnw322 nw322 0 2f
CT1115 t1115 0 0.1f
CT1116 t1116 0 0.1f
CT1117 t1117 0 0.1f
M2873 t1115 nw222 vdd vdd pch w=2u l=180n
M2874 t1115 nq69 vdd vdd pch w=2u l=180n
CT1118 t1118 0 0.1f
M2875 t1115 nw222 t1118 0 nch w=1u l=180n
M2876 t1118 nq69 0 0 nch w=1u l=180n
M2877 t1116 nw222 vdd vdd pch w=2u l=180n
M2878 t1116 t1115 vdd vdd pch w=2u l=180n
CT1119 t1119 0 0.1f
M2879 t1116 nw222 t1119 0 nch w=1u l=180n
M2880 t1119 t1115 0 0 nch w=1u l=180n
M2881 t1117 nq69 vdd vdd pch w=2u l=180n
M2882 t1117 t1115 vdd vdd pch w=2u l=180n
CT1120 t1120 0 0.1f
M2883 t1117 nq69 t1120 0 nch w=1u l=180n
M2884 t1120 t1115 0 0 nch w=1u l=180n
M2885 nw323 t1116 vdd vdd pch w=2u l=180n
M2886 nw323 t1117 vdd vdd pch w=2u l=180n
CT1121 t1121 0 0.1f
M2887 nw323 t1116 t1121 0 nch w=1u l=180n
M2888 t1121 t1117 0 0 nch w=1u l=180n
Cnw323 nw323 0 2f
M2889 nw324 nw225 vdd vdd pch w=2u l=180n
M2890 nw324 nq73 vdd vdd pch w=2u l=180n
CT1122 t1122 0 0.1f
M2891 nw324 nw225 t1122 0 nch w=1u l=180n
M2892 t1122 nq73 0 0 nch w=1u l=180n
Cnw324 nw324 0 2f
M2893 nw325 nw228 0 0 nch w=1u l=180n
M2894 nw325 ni3 0 0 nch w=1u l=180n
CT1123 t1123 0 0.1f
M2895 t1123 nw228 vdd vdd pch w=2u l=180n
M2896 nw325 ni3 t1123 vdd pch w=2u l=180n
Cnw325 nw325 0 2f
CT1124 t1124 0 0.1f
M2897 t1124 nw231 vdd vdd pch w=2u l=180n
M2898 t1124 ni7 vdd vdd pch w=2u l=180n
CT1125 t1125 0 0.1f
M2899 t1124 nw231 t1125 0 nch w=1u l=180n
M2900 t1125 ni7 0 0 nch w=1u l=180n
M2901 nw326 t1124 vdd vdd pch w=2u l=180n
M2902 nw326 t1124 0 0 nch w=1u l=180n
Cnw326 nw326 0 2f
CT1126 t1126 0 0.1f
M2903 t1126 nw234 0 0 nch w=1u l=180n
M2904 t1126 ni11 0 0 nch w=1u l=180n
CT1127 t1127 0 0.1f
M2905 t1127 nw234 vdd vdd pch w=2u l=180n
M2906 t1126 ni11 t1127 vdd pch w=2u l=180n
M2907 nw327 t1126 vdd vdd pch w=2u l=180n
M2908 nw327 t1126 0 0 nch w=1u l=180n
Cnw327 nw327 0 2f
CT1128 t1128 0 0.1f
CT1129 t1129 0 0.1f
CT1130 t1130 0 0.1f
M2909 t1128 nw237 vdd vdd pch w=2u l=180n
M2910 t1128 ni15 vdd vdd pch w=2u l=180n
CT1131 t1131 0 0.1f
M2911 t1128 nw237 t1131 0 nch w=1u l=180n
M2912 t1131 ni15 0 0 nch w=1u l=180n
M2913 t1129 nw237 vdd vdd pch w=2u l=180n
M2914 t1129 t1128 vdd vdd pch w=2u l=180n
CT1132 t1132 0 0.1f
M2915 t1129 nw237 t1132 0 nch w=1u l=180n
M2916 t1132 t1128 0 0 nch w=1u l=180n
M2917 t1130 ni15 vdd vdd pch w=2u l=180n
M2918 t1130 t1128 vdd vdd pch w=2u l=180n
CT1133 t1133 0 0.1f
M2919 t1130 ni15 t1133 0 nch w=1u l=180n
M2920 t1133 t1128 0 0 nch w=1u l=180n
M2921 nw328 t1129 vdd vdd pch w=2u l=180n
M2922 nw328 t1130 vdd vdd pch w=2u l=180n
CT1134 t1134 0 0.1f
M2923 nw328 t1129 t1134 0 nch w=1u l=180n
M2924 t1134 t1130 0 0 nch w=1u l=180n
Cnw328 nw328 0 2f
M2925 nw329 nw240 vdd vdd pch w=2u l=180n
M2926 nw329 nw152 vdd vdd pch w=2u l=180n
CT1135 t1135 0 0.1f
M2927 nw329 nw240 t1135 0 nch w=1u l=180n
M2928 t1135 nw152 0 0 nch w=1u l=180n
Cnw329 nw329 0 2f
M2929 nw330 nw243 0 0 nch w=1u l=180n
M2930 nw330 nw156 0 0 nch w=1u l=180n
CT1136 t1136 0 0.1f
M2931 t1136 nw243 vdd vdd pch w=2u l=180n
M2932 nw330 nw156 t1136 vdd pch w=2u l=180n
Cnw330 nw330 0 2f
CT1137 t1137 0 0.1f
M2933 t1137 nw246 vdd vdd pch w=2u l=180n
M2934 t1137 nw160 vdd vdd pch w=2u l=180n
CT1138 t1138 0 0.1f
M2935 t1137 nw246 t1138 0 nch w=1u l=180n
M2936 t1138 nw160 0 0 nch w=1u l=180n
M2937 nw331 t1137 vdd vdd pch w=2u l=180n
M2938 nw331 t1137 0 0 nch w=1u l=180n
Cnw331 nw331 0 2f
CT1139 t1139 0 0.1f
M2939 t1139 nw249 0 0 nch w=1u l=180n
M2940 t1139 nw164 0 0 nch w=1u l=180n
CT1140 t1140 0 0.1f
M2941 t1140 nw249 vdd vdd pch w=2u l=180n
M2942 t1139 nw164 t1140 vdd pch w=2u l=180n
M2943 nw332 t1139 vdd vdd pch w=2u l=180n
M2944 nw332 t1139 0 0 nch w=1u l=180n
Cnw332 nw332 0 2f
CT1141 t1141 0 0.1f
CT1142 t1142 0 0.1f
CT1143 t1143 0 0.1f
M2945 t1141 nw252 vdd vdd pch w=2u l=180n
M2946 t1141 nw168 vdd vdd pch w=2u l=180n
CT1144 t1144 0 0.1f
M2947 t1141 nw252 t1144 0 nch w=1u l=180n
M2948 t1144 nw168 0 0 nch w=1u l=180n
M2949 t1142 nw252 vdd vdd pch w=2u l=180n
M2950 t1142 t1141 vdd vdd pch w=2u l=180n
CT1145 t1145 0 0.1f
M2951 t1142 nw252 t1145 0 nch w=1u l=180n
M2952 t1145 t1141 0 0 nch w=1u l=180n
M2953 t1143 nw168 vdd vdd pch w=2u l=180n
M2954 t1143 t1141 vdd vdd pch w=2u l=180n
CT1146 t1146 0 0.1f
M2955 t1143 nw168 t1146 0 nch w=1u l=180n
M2956 t1146 t1141 0 0 nch w=1u l=180n
M2957 nw333 t1142 vdd vdd pch w=2u l=180n
M2958 nw333 t1143 vdd vdd pch w=2u l=180n
CT1147 t1147 0 0.1f
M2959 nw333 t1142 t1147 0 nch w=1u l=180n
M2960 t1147 t1143 0 0 nch w=1u l=180n
Cnw333 nw333 0 2f
M2961 nw334 nw255 vdd vdd pch w=2u l=180n
M2962 nw334 nw172 vdd vdd pch w=2u l=180n
CT1148 t1148 0 0.1f
M2963 nw334 nw255 t1148 0 nch w=1u l=180n
M2964 t1148 nw172 0 0 nch w=1u l=180n
Cnw334 nw334 0 2f
M2965 nw335 nw258 0 0 nch w=1u l=180n
M2966 nw335 nw176 0 0 nch w=1u l=180n
CT1149 t1149 0 0.1f
M2967 t1149 nw258 vdd vdd pch w=2u l=180n
M2968 nw335 nw176 t1149 vdd pch w=2u l=180n
Cnw335 nw335 0 2f
CT1150 t1150 0 0.1f
M2969 t1150 nw261 vdd vdd pch w=2u l=180n
M2970 t1150 nw180 vdd vdd pch w=2u l=180n
CT1151 t1151 0 0.1f
M2971 t1150 nw261 t1151 0 nch w=1u l=180n
M2972 t1151 nw180 0 0 nch w=1u l=180n
M2973 nw336 t1150 vdd vdd pch w=2u l=180n
M2974 nw336 t1150 0 0 nch w=1u l=180n
Cnw336 nw336 0 2f
CT1152 t1152 0 0.1f
M2975 t1152 nw264 0 0 nch w=1u l=180n
M2976 t1152 nw184 0 0 nch w=1u l=180n
CT1153 t1153 0 0.1f
M2977 t1153 nw264 vdd vdd pch w=2u l=180n
M2978 t1152 nw184 t1153 vdd pch w=2u l=180n
M2979 nw337 t1152 vdd vdd pch w=2u l=180n
M2980 nw337 t1152 0 0 nch w=1u l=180n
Cnw337 nw337 0 2f
CT1154 t1154 0 0.1f
CT1155 t1155 0 0.1f
CT1156 t1156 0 0.1f
M2981 t1154 nw267 vdd vdd pch w=2u l=180n
M2982 t1154 nw188 vdd vdd pch w=2u l=180n
CT1157 t1157 0 0.1f
M2983 t1154 nw267 t1157 0 nch w=1u l=180n
M2984 t1157 nw188 0 0 nch w=1u l=180n
M2985 t1155 nw267 vdd vdd pch w=2u l=180n
M2986 t1155 t1154 vdd vdd pch w=2u l=180n
CT1158 t1158 0 0.1f
M2987 t1155 nw267 t1158 0 nch w=1u l=180n
M2988 t1158 t1154 0 0 nch w=1u l=180n
M2989 t1156 nw188 vdd vdd pch w=2u l=180n
M2990 t1156 t1154 vdd vdd pch w=2u l=180n
CT1159 t1159 0 0.1f
M2991 t1156 nw188 t1159 0 nch w=1u l=180n
M2992 t1159 t1154 0 0 nch w=1u l=180n
M2993 nw338 t1155 vdd vdd pch w=2u l=180n
M2994 nw338 t1156 vdd vdd pch w=2u l=180n
CT1160 t1160 0 0.1f
M2995 nw338 t1155 t1160 0 nch w=1u l=180n
M2996 t1160 t1156 0 0 nch w=1u l=180n
Cnw338 nw338 0 2f
M2997 nw339 nw270 vdd vdd pch w=2u l=180n
M2998 nw339 nw192 vdd vdd pch w=2u l=180n
CT1161 t1161 0 0.1f
M2999 nw339 nw270 t1161 0 nch w=1u l=180n
M3000 t1161 nw192 0 0 nch w=1u l=180n
Cnw339 nw339 0 2f
M3001 nw340 nw273 0 0 nch w=1u l=180n
M3002 nw340 nw196 0 0 nch w=1u l=180n
CT1162 t1162 0 0.1f
M3003 t1162 nw273 vdd vdd pch w=2u l=180n
M3004 nw340 nw196 t1162 vdd pch w=2u l=180n
Cnw340 nw340 0 2f
CT1163 t1163 0 0.1f
M3005 t1163 nw276 vdd vdd pch w=2u l=180n
M3006 t1163 nw200 vdd vdd pch w=2u l=180n
CT1164 t1164 0 0.1f
M3007 t1163 nw276 t1164 0 nch w=1u l=180n
M3008 t1164 nw200 0 0 nch w=1u l=180n
M3009 nw341 t1163 vdd vdd pch w=2u l=180n
M3010 nw341 t1163 0 0 nch w=1u l=180n
Cnw341 nw341 0 2f
CT1165 t1165 0 0.1f
M3011 t1165 nw279 0 0 nch w=1u l=180n
M3012 t1165 nw204 0 0 nch w=1u l=180n
CT1166 t1166 0 0.1f
M3013 t1166 nw279 vdd vdd pch w=2u l=180n
M3014 t1165 nw204 t1166 vdd pch w=2u l=180n
M3015 nw342 t1165 vdd vdd pch w=2u l=180n
M3016 nw342 t1165 0 0 nch w=1u l=180n
Cnw342 nw342 0 2f
CT1167 t1167 0 0.1f
CT1168 t1168 0 0.1f
CT1169 t1169 0 0.1f
M3017 t1167 nw282 vdd vdd pch w=2u l=180n
M3018 t1167 nw208 vdd vdd pch w=2u l=180n
CT1170 t1170 0 0.1f
M3019 t1167 nw282 t1170 0 nch w=1u l=180n
M3020 t1170 nw208 0 0 nch w=1u l=180n
M3021 t1168 nw282 vdd vdd pch w=2u l=180n
M3022 t1168 t1167 vdd vdd pch w=2u l=180n
CT1171 t1171 0 0.1f
M3023 t1168 nw282 t1171 0 nch w=1u l=180n
M3024 t1171 t1167 0 0 nch w=1u l=180n
M3025 t1169 nw208 vdd vdd pch w=2u l=180n
M3026 t1169 t1167 vdd vdd pch w=2u l=180n
CT1172 t1172 0 0.1f
M3027 t1169 nw208 t1172 0 nch w=1u l=180n
M3028 t1172 t1167 0 0 nch w=1u l=180n
M3029 nw343 t1168 vdd vdd pch w=2u l=180n
M3030 nw343 t1169 vdd vdd pch w=2u l=180n
CT1173 t1173 0 0.1f
M3031 nw343 t1168 t1173 0 nch w=1u l=180n
M3032 t1173 t1169 0 0 nch w=1u l=180n
Cnw343 nw343 0 2f
M3033 nw344 nw285 vdd vdd pch w=2u l=180n
M3034 nw344 nw212 vdd vdd pch w=2u l=180n
CT1174 t1174 0 0.1f
M3035 nw344 nw285 t1174 0 nch w=1u l=180n
M3036 t1174 nw212 0 0 nch w=1u l=180n
Cnw344 nw344 0 2f
M3037 nw345 nw288 0 0 nch w=1u l=180n
M3038 nw345 nw216 0 0 nch w=1u l=180n
CT1175 t1175 0 0.1f
M3039 t1175 nw288 vdd vdd pch w=2u l=180n
M3040 nw345 nw216 t1175 vdd pch w=2u l=180n
Cnw345 nw345 0 2f
CT1176 t1176 0 0.1f
M3041 t1176 nw291 vdd vdd pch w=2u l=180n
M3042 t1176 nw220 vdd vdd pch w=2u l=180n
CT1177 t1177 0 0.1f
M3043 t1176 nw291 t1177 0 nch w=1u l=180n
M3044 t1177 nw220 0 0 nch w=1u l=180n
M3045 nw346 t1176 vdd vdd pch w=2u l=180n
M3046 nw346 t1176 0 0 nch w=1u l=180n
Cnw346 nw346 0 2f
CT1178 t1178 0 0.1f
M3047 t1178 nw294 0 0 nch w=1u l=180n
M3048 t1178 nw224 0 0 nch w=1u l=180n
CT1179 t1179 0 0.1f
M3049 t1179 nw294 vdd vdd pch w=2u l=180n
M3050 t1178 nw224 t1179 vdd pch w=2u l=180n
M3051 nw347 t1178 vdd vdd pch w=2u l=180n
M3052 nw347 t1178 0 0 nch w=1u l=180n
Cnw347 nw347 0 2f
CT1180 t1180 0 0.1f
CT1181 t1181 0 0.1f
CT1182 t1182 0 0.1f
M3053 t1180 nw297 vdd vdd pch w=2u l=180n
M3054 t1180 nw228 vdd vdd pch w=2u l=180n
CT1183 t1183 0 0.1f
M3055 t1180 nw297 t1183 0 nch w=1u l=180n
M3056 t1183 nw228 0 0 nch w=1u l=180n
M3057 t1181 nw297 vdd vdd pch w=2u l=180n
M3058 t1181 t1180 vdd vdd pch w=2u l=180n
CT1184 t1184 0 0.1f
M3059 t1181 nw297 t1184 0 nch w=1u l=180n
M3060 t1184 t1180 0 0 nch w=1u l=180n
M3061 t1182 nw228 vdd vdd pch w=2u l=180n
M3062 t1182 t1180 vdd vdd pch w=2u l=180n
CT1185 t1185 0 0.1f
M3063 t1182 nw228 t1185 0 nch w=1u l=180n
M3064 t1185 t1180 0 0 nch w=1u l=180n
M3065 nw348 t1181 vdd vdd pch w=2u l=180n
M3066 nw348 t1182 vdd vdd pch w=2u l=180n
CT1186 t1186 0 0.1f
M3067 nw348 t1181 t1186 0 nch w=1u l=180n
M3068 t1186 t1182 0 0 nch w=1u l=180n
Cnw348 nw348 0 2f
M3069 nw349 nw300 vdd vdd pch w=2u l=180n
M3070 nw349 nw232 vdd vdd pch w=2u l=180n
CT1187 t1187 0 0.1f
M3071 nw349 nw300 t1187 0 nch w=1u l=180n
M3072 t1187 nw232 0 0 nch w=1u l=180n
Cnw349 nw349 0 2f
M3073 nw350 nw303 0 0 nch w=1u l=180n
M3074 nw350 nw236 0 0 nch w=1u l=180n
CT1188 t1188 0 0.1f
M3075 t1188 nw303 vdd vdd pch w=2u l=180n
M3076 nw350 nw236 t1188 vdd pch w=2u l=180n
Cnw350 nw350 0 2f
CT1189 t1189 0 0.1f
M3077 t1189 nw306 vdd vdd pch w=2u l=180n
M3078 t1189 nw240 vdd vdd pch w=2u l=180n
CT1190 t1190 0 0.1f
M3079 t1189 nw306 t1190 0 nch w=1u l=180n
M3080 t1190 nw240 0 0 nch w=1u l=180n
M3081 nw351 t1189 vdd vdd pch w=2u l=180n
M3082 nw351 t1189 0 0 nch w=1u l=180n
Cnw351 nw351 0 2f
CT1191 t1191 0 0.1f
M3083 t1191 nw309 0 0 nch w=1u l=180n
M3084 t1191 nw244 0 0 nch w=1u l=180n
CT1192 t1192 0 0.1f
M3085 t1192 nw309 vdd vdd pch w=2u l=180n
M3086 t1191 nw244 t1192 vdd pch w=2u l=180n
M3087 nw352 t1191 vdd vdd pch w=2u l=180n
M3088 nw352 t1191 0 0 nch w=1u l=180n
Cnw352 nw352 0 2f
CT1193 t1193 0 0.1f
CT1194 t1194 0 0.1f
CT1195 t1195 0 0.1f
M3089 t1193 nw312 vdd vdd pch w=2u l=180n
M3090 t1193 nw248 vdd vdd pch w=2u l=180n
CT1196 t1196 0 0.1f
M3091 t1193 nw312 t1196 0 nch w=1u l=180n
M3092 t1196 nw248 0 0 nch w=1u l=180n
M3093 t1194 nw312 vdd vdd pch w=2u l=180n
M3094 t1194 t1193 vdd vdd pch w=2u l=180n
CT1197 t1197 0 0.1f
M3095 t1194 nw312 t1197 0 nch w=1u l=180n
M3096 t1197 t1193 0 0 nch w=1u l=180n
M3097 t1195 nw248 vdd vdd pch w=2u l=180n
M3098 t1195 t1193 vdd vdd pch w=2u l=180n
CT1198 t1198 0 0.1f
M3099 t1195 nw248 t1198 0 nch w=1u l=180n
M3100 t1198 t1193 0 0 nch w=1u l=180n
M3101 nw353 t1194 vdd vdd pch w=2u l=180n
M3102 nw353 t1195 vdd vdd pch w=2u l=180n
CT1199 t1199 0 0.1f
M3103 nw353 t1194 t1199 0 nch w=1u l=180n
M3104 t1199 t1195 0 0 nch w=1u l=180n
Cnw353 nw353 0 2f
M3105 nw354 nw315 vdd vdd pch w=2u l=180n
M3106 nw354 nw252 vdd vdd pch w=2u l=180n
CT1200 t1200 0 0.1f
M3107 nw354 nw315 t1200 0 nch w=1u l=180n
M3108 t1200 nw252 0 0 nch w=1u l=180n
Cnw354 nw354 0 2f
M3109 nw355 nw318 0 0 nch w=1u l=180n
M3110 nw355 nw256 0 0 nch w=1u l=180n
CT1201 t1201 0 0.1f
M3111 t1201 nw318 vdd vdd pch w=2u l=180n
M3112 nw355 nw256 t1201 vdd pch w=2u l=180n
Cnw355 nw355 0 2f
CT1202 t1202 0 0.1f
M3113 t1202 nw321 vdd vdd pch w=2u l=180n
M3114 t1202 nw260 vdd vdd pch w=2u l=180n
CT1203 t1203 0 0.1f
M3115 t1202 nw321 t1203 0 nch w=1u l=180n
M3116 t1203 nw260 0 0 nch w=1u l=180n
M3117 nw356 t1202 vdd vdd pch w=2u l=180n
M3118 nw356 t1202 0 0 nch w=1u l=180n
Cnw356 nw356 0 2f
CT1204 t1204 0 0.1f
M3119 t1204 nw324 0 0 nch w=1u l=180n
M3120 t1204 nw264 0 0 nch w=1u l=180n
CT1205 t1205 0 0.1f
M3121 t1205 nw324 vdd vdd pch w=2u l=180n
M3122 t1204 nw264 t1205 vdd pch w=2u l=180n
M3123 nw357 t1204 vdd vdd pch w=2u l=180n
M3124 nw357 t1204 0 0 nch w=1u l=180n
Cnw357 nw357 0 2f
CT1206 t1206 0 0.1f
CT1207 t1207 0 0.1f
CT1208 t1208 0 0.1f
M3125 t1206 nw327 vdd vdd pch w=2u l=180n
M3126 t1206 nw268 vdd vdd pch w=2u l=180n
CT1209 t1209 0 0.1f
M3127 t1206 nw327 t1209 0 nch w=1u l=180n
M3128 t1209 nw268 0 0 nch w=1u l=180n
M3129 t1207 nw327 vdd vdd pch w=2u l=180n
M3130 t1207 t1206 vdd vdd pch w=2u l=180n
CT1210 t1210 0 0.1f
M3131 t1207 nw327 t1210 0 nch w=1u l=180n
M3132 t1210 t1206 0 0 nch w=1u l=180n
M3133 t1208 nw268 vdd vdd pch w=2u l=180n
M3134 t1208 t1206 vdd vdd pch w=2u l=180n
CT1211 t1211 0 0.1f
M3135 t1208 nw268 t1211 0 nch w=1u l=180n
M3136 t1211 t1206 0 0 nch w=1u l=180n
M3137 nw358 t1207 vdd vdd pch w=2u l=180n
M3138 nw358 t1208 vdd vdd pch w=2u l=180n
CT1212 t1212 0 0.1f
M3139 nw358 t1207 t1212 0 nch w=1u l=180n
M3140 t1212 t1208 0 0 nch w=1u l=180n
Cnw358 nw358 0 2f
M3141 nw359 nw330 vdd vdd pch w=2u l=180n
M3142 nw359 nw272 vdd vdd pch w=2u l=180n
CT1213 t1213 0 0.1f
M3143 nw359 nw330 t1213 0 nch w=1u l=180n
M3144 t1213 nw272 0 0 nch w=1u l=180n
Cnw359 nw359 0 2f
M3145 nw360 nw333 0 0 nch w=1u l=180n
M3146 nw360 nw276 0 0 nch w=1u l=180n
CT1214 t1214 0 0.1f
M3147 t1214 nw333 vdd vdd pch w=2u l=180n
M3148 nw360 nw276 t1214 vdd pch w=2u l=180n
Cnw360 nw360 0 2f
CT1215 t1215 0 0.1f
M3149 t1215 nw336 vdd vdd pch w=2u l=180n
M3150 t1215 nw280 vdd vdd pch w=2u l=180n
CT1216 t1216 0 0.1f
M3151 t1215 nw336 t1216 0 nch w=1u l=180n
M3152 t1216 nw280 0 0 nch w=1u l=180n
M3153 nw361 t1215 vdd vdd pch w=2u l=180n
M3154 nw361 t1215 0 0 nch w=1u l=180n
Cnw361 nw361 0 2f
CT1217 t1217 0 0.1f
M3155 t1217 nw339 0 0 nch w=1u l=180n
M3156 t1217 nw284 0 0 nch w=1u l=180n
CT1218 t1218 0 0.1f
M3157 t1218 nw339 vdd vdd pch w=2u l=180n
M3158 t1217 nw284 t1218 vdd pch w=2u l=180n
M3159 nw362 t1217 vdd vdd pch w=2u l=180n
M3160 nw362 t1217 0 0 nch w=1u l=180n
Cnw362 nw362 0 2f
CT1219 t1219 0 0.1f
CT1220 t1220 0 0.1f
CT1221 t1221 0 0.1f
M3161 t1219 nw342 vdd vdd pch w=2u l=180n
M3162 t1219 nw288 vdd vdd pch w=2u l=180n
CT1222 t1222 0 0.1f
M3163 t1219 nw342 t1222 0 nch w=1u l=180n
M3164 t1222 nw288 0 0 nch w=1u l=180n
M3165 t1220 nw342 vdd vdd pch w=2u l=180n
M3166 t1220 t1219 vdd vdd pch w=2u l=180n
CT1223 t1223 0 0.1f
M3167 t1220 nw342 t1223 0 nch w=1u l=180n
M3168 t1223 t1219 0 0 nch w=1u l=180n
M3169 t1221 nw288 vdd vdd pch w=2u l=180n
M3170 t1221 t1219 vdd vdd pch w=2u l=180n
CT1224 t1224 0 0.1f
M3171 t1221 nw288 t1224 0 nch w=1u l=180n
M3172 t1224 t1219 0 0 nch w=1u l=180n
M3173 nw363 t1220 vdd vdd pch w=2u l=180n
M3174 nw363 t1221 vdd vdd pch w=2u l=180n
CT1225 t1225 0 0.1f
M3175 nw363 t1220 t1225 0 nch w=1u l=180n
M3176 t1225 t1221 0 0 nch w=1u l=180n
Cnw363 nw363 0 2f
M3177 nw364 nw345 vdd vdd pch w=2u l=180n
M3178 nw364 nw292 vdd vdd pch w=2u l=180n
CT1226 t1226 0 0.1f
M3179 nw364 nw345 t1226 0 nch w=1u l=180n
M3180 t1226 nw292 0 0 nch w=1u l=180n
Cnw364 nw364 0 2f
M3181 nw365 nw348 0 0 nch w=1u l=180n
M3182 nw365 nw296 0 0 nch w=1u l=180n
CT1227 t1227 0 0.1f
M3183 t1227 nw348 vdd vdd pch w=2u l=180n
M3184 nw365 nw296 t1227 vdd pch w=2u l=180n
Cnw365 nw365 0 2f
CT1228 t1228 0 0.1f
M3185 t1228 nw351 vdd vdd pch w=2u l=180n
M3186 t1228 nw300 vdd vdd pch w=2u l=180n
CT1229 t1229 0 0.1f
M3187 t1228 nw351 t1229 0 nch w=1u l=180n
M3188 t1229 nw300 0 0 nch w=1u l=180n
M3189 nw366 t1228 vdd vdd pch w=2u l=180n
M3190 nw366 t1228 0 0 nch w=1u l=180n
Cnw366 nw366 0 2f
CT1230 t1230 0 0.1f
M3191 t1230 nw354 0 0 nch w=1u l=180n
M3192 t1230 nw304 0 0 nch w=1u l=180n
CT1231 t1231 0 0.1f
M3193 t1231 nw354 vdd vdd pch w=2u l=180n
M3194 t1230 nw304 t1231 vdd pch w=2u l=180n
M3195 nw367 t1230 vdd vdd pch w=2u l=180n
M3196 nw367 t1230 0 0 nch w=1u l=180n
Cnw367 nw367 0 2f
CT1232 t1232 0 0.1f
CT1233 t1233 0 0.1f
CT1234 t1234 0 0.1f
M3197 t1232 nw357 vdd vdd pch w=2u l=180n
M3198 t1232 nw308 vdd vdd pch w=2u l=180n
CT1235 t1235 0 0.1f
M3199 t1232 nw357 t1235 0 nch w=1u l=180n
M3200 t1235 nw308 0 0 nch w=1u l=180n
M3201 t1233 nw357 vdd vdd pch w=2u l=180n
M3202 t1233 t1232 vdd vdd pch w=2u l=180n
CT1236 t1236 0 0.1f
M3203 t1233 nw357 t1236 0 nch w=1u l=180n
M3204 t1236 t1232 0 0 nch w=1u l=180n
M3205 t1234 nw308 vdd vdd pch w=2u l=180n
M3206 t1234 t1232 vdd vdd pch w=2u l=180n
CT1237 t1237 0 0.1f
M3207 t1234 nw308 t1237 0 nch w=1u l=180n
M3208 t1237 t1232 0 0 nch w=1u l=180n
M3209 nw368 t1233 vdd vdd pch w=2u l=180n
M3210 nw368 t1234 vdd vdd pch w=2u l=180n
CT1238 t1238 0 0.1f
M3211 nw368 t1233 t1238 0 nch w=1u l=180n
M3212 t1238 t1234 0 0 nch w=1u l=180n
Cnw368 nw368 0 2f
M3213 nw369 nw360 vdd vdd pch w=2u l=180n
M3214 nw369 nw312 vdd vdd pch w=2u l=180n
CT1239 t1239 0 0.1f
M3215 nw369 nw360 t1239 0 nch w=1u l=180n
M3216 t1239 nw312 0 0 nch w=1u l=180n
Cnw369 nw369 0 2f
M3217 nw370 nw363 0 0 nch w=1u l=180n
M3218 nw370 nw316 0 0 nch w=1u l=180n
CT1240 t1240 0 0.1f
M3219 t1240 nw363 vdd vdd pch w=2u l=180n
M3220 nw370 nw316 t1240 vdd pch w=2u l=180n
Cnw370 nw370 0 2f
CT1241 t1241 0 0.1f
M3221 t1241 nw366 vdd vdd pch w=2u l=180n
M3222 t1241 nw320 vdd vdd pch w=2u l=180n
CT1242 t1242 0 0.1f
M3223 t1241 nw366 t1242 0 nch w=1u l=180n
M3224 t1242 nw320 0 0 nch w=1u l=180n
M3225 nw371 t1241 vdd vdd pch w=2u l=180n
M3226 nw371 t1241 0 0 nch w=1u l=180n
Cnw371 nw371 0 2f
CT1243 t1243 0 0.1f
M3227 t1243 nw369 0 0 nch w=1u l=180n
M3228 t1243 nw324 0 0 nch w=1u l=180n
CT1244 t1244 0 0.1f
M3229 t1244 nw369 vdd vdd pch w=2u l=180n
M3230 t1243 nw324 t1244 vdd pch w=2u l=180n
M3231 nw372 t1243 vdd vdd pch w=2u l=180n
M3232 nw372 t1243 0 0 nch w=1u l=180n
Cnw372 nw372 0 2f
CT1245 t1245 0 0.1f
CT1246 t1246 0 0.1f
CT1247 t1247 0 0.1f
M3233 t1245 nw372 vdd vdd pch w=2u l=180n
M3234 t1245 nw328 vdd vdd pch w=2u l=180n
CT1248 t1248 0 0.1f
M3235 t1245 nw372 t1248 0 nch w=1u l=180n
M3236 t1248 nw328 0 0 nch w=1u l=180n
M3237 t1246 nw372 vdd vdd pch w=2u l=180n
M3238 t1246 t1245 vdd vdd pch w=2u l=180n
CT1249 t1249 0 0.1f
M3239 t1246 nw372 t1249 0 nch w=1u l=180n
M3240 t1249 t1245 0 0 nch w=1u l=180n
M3241 t1247 nw328 vdd vdd pch w=2u l=180n
M3242 t1247 t1245 vdd vdd pch w=2u l=180n
CT1250 t1250 0 0.1f
M3243 t1247 nw328 t1250 0 nch w=1u l=180n
M3244 t1250 t1245 0 0 nch w=1u l=180n
M3245 nw373 t1246 vdd vdd pch w=2u l=180n
M3246 nw373 t1247 vdd vdd pch w=2u l=180n
CT1251 t1251 0 0.1f
M3247 nw373 t1246 t1251 0 nch w=1u l=180n
M3248 t1251 t1247 0 0 nch w=1u l=180n
Cnw373 nw373 0 2f
M3249 nw374 nq1 vdd vdd pch w=2u l=180n
M3250 nw374 nw332 vdd vdd pch w=2u l=180n
CT1252 t1252 0 0.1f
M3251 nw374 nq1 t1252 0 nch w=1u l=180n
M3252 t1252 nw332 0 0 nch w=1u l=180n
Cnw374 nw374 0 2f
M3253 nw375 nq3 0 0 nch w=1u l=180n
M3254 nw375 nw336 0 0 nch w=1u l=180n
CT1253 t1253 0 0.1f
M3255 t1253 nq3 vdd vdd pch w=2u l=180n
M3256 nw375 nw336 t1253 vdd pch w=2u l=180n
Cnw375 nw375 0 2f
CT1254 t1254 0 0.1f
M3257 t1254 nq5 vdd vdd pch w=2u l=180n
M3258 t1254 nw340 vdd vdd pch w=2u l=180n
CT1255 t1255 0 0.1f
M3259 t1254 nq5 t1255 0 nch w=1u l=180n
M3260 t1255 nw340 0 0 nch w=1u l=180n
M3261 nw376 t1254 vdd vdd pch w=2u l=180n
M3262 nw376 t1254 0 0 nch w=1u l=180n
Cnw376 nw376 0 2f
CT1256 t1256 0 0.1f
M3263 t1256 nq7 0 0 nch w=1u l=180n
M3264 t1256 nw344 0 0 nch w=1u l=180n
CT1257 t1257 0 0.1f
M3265 t1257 nq7 vdd vdd pch w=2u l=180n
M3266 t1256 nw344 t1257 vdd pch w=2u l=180n
M3267 nw377 t1256 vdd vdd pch w=2u l=180n
M3268 nw377 t1256 0 0 nch w=1u l=180n
Cnw377 nw377 0 2f
CT1258 t1258 0 0.1f
CT1259 t1259 0 0.1f
CT1260 t1260 0 0.1f
M3269 t1258 nq9 vdd vdd pch w=2u l=180n
M3270 t1258 nw348 vdd vdd pch w=2u l=180n
CT1261 t1261 0 0.1f
M3271 t1258 nq9 t1261 0 nch w=1u l=180n
M3272 t1261 nw348 0 0 nch w=1u l=180n
M3273 t1259 nq9 vdd vdd pch w=2u l=180n
M3274 t1259 t1258 vdd vdd pch w=2u l=180n
CT1262 t1262 0 0.1f
M3275 t1259 nq9 t1262 0 nch w=1u l=180n
M3276 t1262 t1258 0 0 nch w=1u l=180n
M3277 t1260 nw348 vdd vdd pch w=2u l=180n
M3278 t1260 t1258 vdd vdd pch w=2u l=180n
CT1263 t1263 0 0.1f
M3279 t1260 nw348 t1263 0 nch w=1u l=180n
M3280 t1263 t1258 0 0 nch w=1u l=180n
M3281 nw378 t1259 vdd vdd pch w=2u l=180n
M3282 nw378 t1260 vdd vdd pch w=2u l=180n
CT1264 t1264 0 0.1f
M3283 nw378 t1259 t1264 0 nch w=1u l=180n
M3284 t1264 t1260 0 0 nch w=1u l=180n
Cnw378 nw378 0 2f
M3285 nw379 nq11 vdd vdd pch w=2u l=180n
M3286 nw379 nw352 vdd vdd pch w=2u l=180n
CT1265 t1265 0 0.1f
M3287 nw379 nq11 t1265 0 nch w=1u l=180n
M3288 t1265 nw352 0 0 nch w=1u l=180n
Cnw379 nw379 0 2f
M3289 nw380 nq13 0 0 nch w=1u l=180n
M3290 nw380 nw356 0 0 nch w=1u l=180n
CT1266 t1266 0 0.1f
M3291 t1266 nq13 vdd vdd pch w=2u l=180n
M3292 nw380 nw356 t1266 vdd pch w=2u l=180n
Cnw380 nw380 0 2f
CT1267 t1267 0 0.1f
M3293 t1267 nq15 vdd vdd pch w=2u l=180n
M3294 t1267 nw360 vdd vdd pch w=2u l=180n
CT1268 t1268 0 0.1f
M3295 t1267 nq15 t1268 0 nch w=1u l=180n
M3296 t1268 nw360 0 0 nch w=1u l=180n
M3297 nw381 t1267 vdd vdd pch w=2u l=180n
M3298 nw381 t1267 0 0 nch w=1u l=180n
Cnw381 nw381 0 2f
CT1269 t1269 0 0.1f
M3299 t1269 nq17 0 0 nch w=1u l=180n
M3300 t1269 nw364 0 0 nch w=1u l=180n
CT1270 t1270 0 0.1f
M3301 t1270 nq17 vdd vdd pch w=2u l=180n
M3302 t1269 nw364 t1270 vdd pch w=2u l=180n
M3303 nw382 t1269 vdd vdd pch w=2u l=180n
M3304 nw382 t1269 0 0 nch w=1u l=180n
Cnw382 nw382 0 2f
CT1271 t1271 0 0.1f
CT1272 t1272 0 0.1f
CT1273 t1273 0 0.1f
M3305 t1271 nq19 vdd vdd pch w=2u l=180n
M3306 t1271 nw368 vdd vdd pch w=2u l=180n
CT1274 t1274 0 0.1f
M3307 t1271 nq19 t1274 0 nch w=1u l=180n
M3308 t1274 nw368 0 0 nch w=1u l=180n
M3309 t1272 nq19 vdd vdd pch w=2u l=180n
M3310 t1272 t1271 vdd vdd pch w=2u l=180n
CT1275 t1275 0 0.1f
M3311 t1272 nq19 t1275 0 nch w=1u l=180n
M3312 t1275 t1271 0 0 nch w=1u l=180n
M3313 t1273 nw368 vdd vdd pch w=2u l=180n
M3314 t1273 t1271 vdd vdd pch w=2u l=180n
CT1276 t1276 0 0.1f
M3315 t1273 nw368 t1276 0 nch w=1u l=180n
M3316 t1276 t1271 0 0 nch w=1u l=180n
M3317 nw383 t1272 vdd vdd pch w=2u l=180n
M3318 nw383 t1273 vdd vdd pch w=2u l=180n
CT1277 t1277 0 0.1f
M3319 nw383 t1272 t1277 0 nch w=1u l=180n
M3320 t1277 t1273 0 0 nch w=1u l=180n
Cnw383 nw383 0 2f
M3321 nw384 nq21 vdd vdd pch w=2u l=180n
M3322 nw384 nw372 vdd vdd pch w=2u l=180n
CT1278 t1278 0 0.1f
M3323 nw384 nq21 t1278 0 nch w=1u l=180n
M3324 t1278 nw372 0 0 nch w=1u l=180n
Cnw384 nw384 0 2f
M3325 nw385 nq23 0 0 nch w=1u l=180n
M3326 nw385 nw376 0 0 nch w=1u l=180n
CT1279 t1279 0 0.1f
M3327 t1279 nq23 vdd vdd pch w=2u l=180n
M3328 nw385 nw376 t1279 vdd pch w=2u l=180n
Cnw385 nw385 0 2f
CT1280 t1280 0 0.1f
M3329 t1280 nq25 vdd vdd pch w=2u l=180n
M3330 t1280 nw380 vdd vdd pch w=2u l=180n
CT1281 t1281 0 0.1f
M3331 t1280 nq25 t1281 0 nch w=1u l=180n
M3332 t1281 nw380 0 0 nch w=1u l=180n
M3333 nw386 t1280 vdd vdd pch w=2u l=180n
M3334 nw386 t1280 0 0 nch w=1u l=180n
Cnw386 nw386 0 2f
CT1282 t1282 0 0.1f
M3335 t1282 nq27 0 0 nch w=1u l=180n
M3336 t1282 nw384 0 0 nch w=1u l=180n
CT1283 t1283 0 0.1f
M3337 t1283 nq27 vdd vdd pch w=2u l=180n
M3338 t1282 nw384 t1283 vdd pch w=2u l=180n
M3339 nw387 t1282 vdd vdd pch w=2u l=180n
M3340 nw387 t1282 0 0 nch w=1u l=180n
Cnw387 nw387 0 2f
CT1284 t1284 0 0.1f
CT1285 t1285 0 0.1f
CT1286 t1286 0 0.1f
M3341 t1284 nq29 vdd vdd pch w=2u l=180n
M3342 t1284 nq0 vdd vdd pch w=2u l=180n
CT1287 t1287 0 0.1f
M3343 t1284 nq29 t1287 0 nch w=1u l=180n
M3344 t1287 nq0 0 0 nch w=1u l=180n
M3345 t1285 nq29 vdd vdd pch w=2u l=180n
M3346 t1285 t1284 vdd vdd pch w=2u l=180n
CT1288 t1288 0 0.1f
M3347 t1285 nq29 t1288 0 nch w=1u l=180n
M3348 t1288 t1284 0 0 nch w=1u l=180n
M3349 t1286 nq0 vdd vdd pch w=2u l=180n
M3350 t1286 t1284 vdd vdd pch w=2u l=180n
CT1289 t1289 0 0.1f
M3351 t1286 nq0 t1289 0 nch w=1u l=180n
M3352 t1289 t1284 0 0 nch w=1u l=180n
M3353 nw388 t1285 vdd vdd pch w=2u l=180n
M3354 nw388 t1286 vdd vdd pch w=2u l=180n
CT1290 t1290 0 0.1f
M3355 nw388 t1285 t1290 0 nch w=1u l=180n
M3356 t1290 t1286 0 0 nch w=1u l=180n
Cnw388 nw388 0 2f
M3357 nw389 nq31 vdd vdd pch w=2u l=180n
M3358 nw389 nq3 vdd vdd pch w=2u l=180n
CT1291 t1291 0 0.1f
M3359 nw389 nq31 t1291 0 nch w=1u l=180n
M3360 t1291 nq3 0 0 nch w=1u l=180n
Cnw389 nw389 0 2f
M3361 nw390 nq33 0 0 nch w=1u l=180n
M3362 nw390 nq6 0 0 nch w=1u l=180n
CT1292 t1292 0 0.1f
M3363 t1292 nq33 vdd vdd pch w=2u l=180n
M3364 nw390 nq6 t1292 vdd pch w=2u l=180n
Cnw390 nw390 0 2f
CT1293 t1293 0 0.1f
M3365 t1293 nq35 vdd vdd pch w=2u l=180n
M3366 t1293 nq9 vdd vdd pch w=2u l=180n
CT1294 t1294 0 0.1f
M3367 t1293 nq35 t1294 0 nch w=1u l=180n
M3368 t1294 nq9 0 0 nch w=1u l=180n
M3369 nw391 t1293 vdd vdd pch w=2u l=180n
M3370 nw391 t1293 0 0 nch w=1u l=180n
Cnw391 nw391 0 2f
CT1295 t1295 0 0.1f
M3371 t1295 nq37 0 0 nch w=1u l=180n
M3372 t1295 nq12 0 0 nch w=1u l=180n
CT1296 t1296 0 0.1f
M3373 t1296 nq37 vdd vdd pch w=2u l=180n
M3374 t1295 nq12 t1296 vdd pch w=2u l=180n
M3375 nw392 t1295 vdd vdd pch w=2u l=180n
M3376 nw392 t1295 0 0 nch w=1u l=180n
Cnw392 nw392 0 2f
CT1297 t1297 0 0.1f
CT1298 t1298 0 0.1f
CT1299 t1299 0 0.1f
M3377 t1297 nq39 vdd vdd pch w=2u l=180n
M3378 t1297 nq15 vdd vdd pch w=2u l=180n
CT1300 t1300 0 0.1f
M3379 t1297 nq39 t1300 0 nch w=1u l=180n
M3380 t1300 nq15 0 0 nch w=1u l=180n
M3381 t1298 nq39 vdd vdd pch w=2u l=180n
M3382 t1298 t1297 vdd vdd pch w=2u l=180n
CT1301 t1301 0 0.1f
M3383 t1298 nq39 t1301 0 nch w=1u l=180n
M3384 t1301 t1297 0 0 nch w=1u l=180n
M3385 t1299 nq15 vdd vdd pch w=2u l=180n
M3386 t1299 t1297 vdd vdd pch w=2u l=180n
CT1302 t1302 0 0.1f
M3387 t1299 nq15 t1302 0 nch w=1u l=180n
M3388 t1302 t1297 0 0 nch w=1u l=180n
M3389 nw393 t1298 vdd vdd pch w=2u l=180n
M3390 nw393 t1299 vdd vdd pch w=2u l=180n
CT1303 t1303 0 0.1f
M3391 nw393 t1298 t1303 0 nch w=1u l=180n
M3392 t1303 t1299 0 0 nch w=1u l=180n
Cnw393 nw393 0 2f
M3393 nw394 nq41 vdd vdd pch w=2u l=180n
M3394 nw394 nq18 vdd vdd pch w=2u l=180n
CT1304 t1304 0 0.1f
M3395 nw394 nq41 t1304 0 nch w=1u l=180n
M3396 t1304 nq18 0 0 nch w=1u l=180n
Cnw394 nw394 0 2f
M3397 nw395 nq43 0 0 nch w=1u l=180n
M3398 nw395 nq21 0 0 nch w=1u l=180n
CT1305 t1305 0 0.1f
M3399 t1305 nq43 vdd vdd pch w=2u l=180n
M3400 nw395 nq21 t1305 vdd pch w=2u l=180n
Cnw395 nw395 0 2f
CT1306 t1306 0 0.1f
M3401 t1306 nq45 vdd vdd pch w=2u l=180n
M3402 t1306 nq24 vdd vdd pch w=2u l=180n
CT1307 t1307 0 0.1f
M3403 t1306 nq45 t1307 0 nch w=1u l=180n
M3404 t1307 nq24 0 0 nch w=1u l=180n
M3405 nw396 t1306 vdd vdd pch w=2u l=180n
M3406 nw396 t1306 0 0 nch w=1u l=180n
Cnw396 nw396 0 2f
CT1308 t1308 0 0.1f
M3407 t1308 nq47 0 0 nch w=1u l=180n
M3408 t1308 nq27 0 0 nch w=1u l=180n
CT1309 t1309 0 0.1f
M3409 t1309 nq47 vdd vdd pch w=2u l=180n
M3410 t1308 nq27 t1309 vdd pch w=2u l=180n
M3411 nw397 t1308 vdd vdd pch w=2u l=180n
M3412 nw397 t1308 0 0 nch w=1u l=180n
Cnw397 nw397 0 2f
CT1310 t1310 0 0.1f
CT1311 t1311 0 0.1f
CT1312 t1312 0 0.1f
M3413 t1310 nq49 vdd vdd pch w=2u l=180n
M3414 t1310 nq30 vdd vdd pch w=2u l=180n
CT1313 t1313 0 0.1f
M3415 t1310 nq49 t1313 0 nch w=1u l=180n
M3416 t1313 nq30 0 0 nch w=1u l=180n
M3417 t1311 nq49 vdd vdd pch w=2u l=180n
M3418 t1311 t1310 vdd vdd pch w=2u l=180n
CT1314 t1314 0 0.1f
M3419 t1311 nq49 t1314 0 nch w=1u l=180n
M3420 t1314 t1310 0 0 nch w=1u l=180n
M3421 t1312 nq30 vdd vdd pch w=2u l=180n
M3422 t1312 t1310 vdd vdd pch w=2u l=180n
CT1315 t1315 0 0.1f
M3423 t1312 nq30 t1315 0 nch w=1u l=180n
M3424 t1315 t1310 0 0 nch w=1u l=180n
M3425 nw398 t1311 vdd vdd pch w=2u l=180n
M3426 nw398 t1312 vdd vdd pch w=2u l=180n
CT1316 t1316 0 0.1f
M3427 nw398 t1311 t1316 0 nch w=1u l=180n
M3428 t1316 t1312 0 0 nch w=1u l=180n
Cnw398 nw398 0 2f
M3429 nw399 nq51 vdd vdd pch w=2u l=180n
M3430 nw399 nq33 vdd vdd pch w=2u l=180n
CT1317 t1317 0 0.1f
M3431 nw399 nq51 t1317 0 nch w=1u l=180n
M3432 t1317 nq33 0 0 nch w=1u l=180n
Cnw399 nw399 0 2f
M3433 nw400 nq53 0 0 nch w=1u l=180n
M3434 nw400 nq36 0 0 nch w=1u l=180n
CT1318 t1318 0 0.1f
M3435 t1318 nq53 vdd vdd pch w=2u l=180n
M3436 nw400 nq36 t1318 vdd pch w=2u l=180n
Cnw400 nw400 0 2f
CT1319 t1319 0 0.1f
M3437 t1319 nq55 vdd vdd pch w=2u l=180n
M3438 t1319 nq39 vdd vdd pch w=2u l=180n
CT1320 t1320 0 0.1f
M3439 t1319 nq55 t1320 0 nch w=1u l=180n
M3440 t1320 nq39 0 0 nch w=1u l=180n
M3441 nw401 t1319 vdd vdd pch w=2u l=180n
M3442 nw401 t1319 0 0 nch w=1u l=180n
Cnw401 nw401 0 2f
CT1321 t1321 0 0.1f
M3443 t1321 nq57 0 0 nch w=1u l=180n
M3444 t1321 nq42 0 0 nch w=1u l=180n
CT1322 t1322 0 0.1f
M3445 t1322 nq57 vdd vdd pch w=2u l=180n
M3446 t1321 nq42 t1322 vdd pch w=2u l=180n
M3447 nw402 t1321 vdd vdd pch w=2u l=180n
M3448 nw402 t1321 0 0 nch w=1u l=180n
Cnw402 nw402 0 2f
CT1323 t1323 0 0.1f
CT1324 t1324 0 0.1f
CT1325 t1325 0 0.1f
M3449 t1323 nq59 vdd vdd pch w=2u l=180n
M3450 t1323 nq45 vdd vdd pch w=2u l=180n
CT1326 t1326 0 0.1f
M3451 t1323 nq59 t1326 0 nch w=1u l=180n
M3452 t1326 nq45 0 0 nch w=1u l=180n
M3453 t1324 nq59 vdd vdd pch w=2u l=180n
M3454 t1324 t1323 vdd vdd pch w=2u l=180n
CT1327 t1327 0 0.1f
M3455 t1324 nq59 t1327 0 nch w=1u l=180n
M3456 t1327 t1323 0 0 nch w=1u l=180n
M3457 t1325 nq45 vdd vdd pch w=2u l=180n
M3458 t1325 t1323 vdd vdd pch w=2u l=180n
CT1328 t1328 0 0.1f
M3459 t1325 nq45 t1328 0 nch w=1u l=180n
M3460 t1328 t1323 0 0 nch w=1u l=180n
M3461 nw403 t1324 vdd vdd pch w=2u l=180n
M3462 nw403 t1325 vdd vdd pch w=2u l=180n
CT1329 t1329 0 0.1f
M3463 nw403 t1324 t1329 0 nch w=1u l=180n
M3464 t1329 t1325 0 0 nch w=1u l=180n
Cnw403 nw403 0 2f
M3465 nw404 nq61 vdd vdd pch w=2u l=180n
M3466 nw404 nq48 vdd vdd pch w=2u l=180n
CT1330 t1330 0 0.1f
M3467 nw404 nq61 t1330 0 nch w=1u l=180n
M3468 t1330 nq48 0 0 nch w=1u l=180n
Cnw404 nw404 0 2f
M3469 nw405 nq63 0 0 nch w=1u l=180n
M3470 nw405 nq51 0 0 nch w=1u l=180n
CT1331 t1331 0 0.1f
M3471 t1331 nq63 vdd vdd pch w=2u l=180n
M3472 nw405 nq51 t1331 vdd pch w=2u l=180n
Cnw405 nw405 0 2f
CT1332 t1332 0 0.1f
M3473 t1332 nq65 vdd vdd pch w=2u l=180n
M3474 t1332 nq54 vdd vdd pch w=2u l=180n
CT1333 t1333 0 0.1f
M3475 t1332 nq65 t1333 0 nch w=1u l=180n
M3476 t1333 nq54 0 0 nch w=1u l=180n
M3477 nw406 t1332 vdd vdd pch w=2u l=180n
M3478 nw406 t1332 0 0 nch w=1u l=180n
Cnw406 nw406 0 2f
CT1334 t1334 0 0.1f
M3479 t1334 nq67 0 0 nch w=1u l=180n
M3480 t1334 nq57 0 0 nch w=1u l=180n
CT1335 t1335 0 0.1f
M3481 t1335 nq67 vdd vdd pch w=2u l=180n
M3482 t1334 nq57 t1335 vdd pch w=2u l=180n
M3483 nw407 t1334 vdd vdd pch w=2u l=180n
M3484 nw407 t1334 0 0 nch w=1u l=180n
Cnw407 nw407 0 2f
CT1336 t1336 0 0.1f
CT1337 t1337 0 0.1f
CT1338 t1338 0 0.1f
M3485 t1336 nq69 vdd vdd pch w=2u l=180n
M3486 t1336 nq60 vdd vdd pch w=2u l=180n
CT1339 t1339 0 0.1f
M3487 t1336 nq69 t1339 0 nch w=1u l=180n
M3488 t1339 nq60 0 0 nch w=1u l=180n
M3489 t1337 nq69 vdd vdd pch w=2u l=180n
M3490 t1337 t1336 vdd vdd pch w=2u l=180n
CT1340 t1340 0 0.1f
M3491 t1337 nq69 t1340 0 nch w=1u l=180n
M3492 t1340 t1336 0 0 nch w=1u l=180n
M3493 t1338 nq60 vdd vdd pch w=2u l=180n
M3494 t1338 t1336 vdd vdd pch w=2u l=180n
CT1341 t1341 0 0.1f
M3495 t1338 nq60 t1341 0 nch w=1u l=180n
M3496 t1341 t1336 0 0 nch w=1u l=180n
M3497 nw408 t1337 vdd vdd pch w=2u l=180n
M3498 nw408 t1338 vdd vdd pch w=2u l=180n
CT1342 t1342 0 0.1f
M3499 nw408 t1337 t1342 0 nch w=1u l=180n
M3500 t1342 t1338 0 0 nch w=1u l=180n
Cnw408 nw408 0 2f
M3501 nw409 nq71 vdd vdd pch w=2u l=180n
M3502 nw409 nq63 vdd vdd pch w=2u l=180n
CT1343 t1343 0 0.1f
M3503 nw409 nq71 t1343 0 nch w=1u l=180n
M3504 t1343 nq63 0 0 nch w=1u l=180n
Cnw409 nw409 0 2f
M3505 nw410 nq73 0 0 nch w=1u l=180n
M3506 nw410 nq66 0 0 nch w=1u l=180n
CT1344 t1344 0 0.1f
M3507 t1344 nq73 vdd vdd pch w=2u l=180n
M3508 nw410 nq66 t1344 vdd pch w=2u l=180n
Cnw410 nw410 0 2f
CT1345 t1345 0 0.1f
M3509 t1345 ni1 vdd vdd pch w=2u l=180n
M3510 t1345 nq69 vdd vdd pch w=2u l=180n
CT1346 t1346 0 0.1f
M3511 t1345 ni1 t1346 0 nch w=1u l=180n
M3512 t1346 nq69 0 0 nch w=1u l=180n
M3513 nw411 t1345 vdd vdd pch w=2u l=180n
M3514 nw411 t1345 0 0 nch w=1u l=180n
Cnw411 nw411 0 2f
CT1347 t1347 0 0.1f
M3515 t1347 ni3 0 0 nch w=1u l=180n
M3516 t1347 nq72 0 0 nch w=1u l=180n
CT1348 t1348 0 0.1f
M3517 t1348 ni3 vdd vdd pch w=2u l=180n
M3518 t1347 nq72 t1348 vdd pch w=2u l=180n
M3519 nw412 t1347 vdd vdd pch w=2u l=180n
M3520 nw412 t1347 0 0 nch w=1u l=180n
Cnw412 nw412 0 2f
CT1349 t1349 0 0.1f
CT1350 t1350 0 0.1f
CT1351 t1351 0 0.1f
M3521 t1349 ni5 vdd vdd pch w=2u l=180n
M3522 t1349 ni1 vdd vdd pch w=2u l=180n
CT1352 t1352 0 0.1f
M3523 t1349 ni5 t1352 0 nch w=1u l=180n
M3524 t1352 ni1 0 0 nch w=1u l=180n
M3525 t1350 ni5 vdd vdd pch w=2u l=180n
M3526 t1350 t1349 vdd vdd pch w=2u l=180n
CT1353 t1353 0 0.1f
M3527 t1350 ni5 t1353 0 nch w=1u l=180n
M3528 t1353 t1349 0 0 nch w=1u l=180n
M3529 t1351 ni1 vdd vdd pch w=2u l=180n
M3530 t1351 t1349 vdd vdd pch w=2u l=180n
CT1354 t1354 0 0.1f
M3531 t1351 ni1 t1354 0 nch w=1u l=180n
M3532 t1354 t1349 0 0 nch w=1u l=180n
M3533 nw413 t1350 vdd vdd pch w=2u l=180n
M3534 nw413 t1351 vdd vdd pch w=2u l=180n
CT1355 t1355 0 0.1f
M3535 nw413 t1350 t1355 0 nch w=1u l=180n
M3536 t1355 t1351 0 0 nch w=1u l=180n
Cnw413 nw413 0 2f
M3537 nw414 ni7 vdd vdd pch w=2u l=180n
M3538 nw414 ni4 vdd vdd pch w=2u l=180n
CT1356 t1356 0 0.1f
M3539 nw414 ni7 t1356 0 nch w=1u l=180n
M3540 t1356 ni4 0 0 nch w=1u l=180n
Cnw414 nw414 0 2f
M3541 nw415 ni9 0 0 nch w=1u l=180n
M3542 nw415 ni7 0 0 nch w=1u l=180n
CT1357 t1357 0 0.1f
M3543 t1357 ni9 vdd vdd pch w=2u l=180n
M3544 nw415 ni7 t1357 vdd pch w=2u l=180n
Cnw415 nw415 0 2f
CT1358 t1358 0 0.1f
M3545 t1358 ni11 vdd vdd pch w=2u l=180n
M3546 t1358 ni10 vdd vdd pch w=2u l=180n
CT1359 t1359 0 0.1f
M3547 t1358 ni11 t1359 0 nch w=1u l=180n
M3548 t1359 ni10 0 0 nch w=1u l=180n
M3549 nw416 t1358 vdd vdd pch w=2u l=180n
M3550 nw416 t1358 0 0 nch w=1u l=180n
Cnw416 nw416 0 2f
CT1360 t1360 0 0.1f
M3551 t1360 ni13 0 0 nch w=1u l=180n
M3552 t1360 nw326 0 0 nch w=1u l=180n
CT1361 t1361 0 0.1f
M3553 t1361 ni13 vdd vdd pch w=2u l=180n
M3554 t1360 nw326 t1361 vdd pch w=2u l=180n
M3555 nw417 t1360 vdd vdd pch w=2u l=180n
M3556 nw417 t1360 0 0 nch w=1u l=180n
Cnw417 nw417 0 2f
CT1362 t1362 0 0.1f
CT1363 t1363 0 0.1f
CT1364 t1364 0 0.1f
M3557 t1362 ni15 vdd vdd pch w=2u l=180n
M3558 t1362 nw149 vdd vdd pch w=2u l=180n
CT1365 t1365 0 0.1f
M3559 t1362 ni15 t1365 0 nch w=1u l=180n
M3560 t1365 nw149 0 0 nch w=1u l=180n
M3561 t1363 ni15 vdd vdd pch w=2u l=180n
M3562 t1363 t1362 vdd vdd pch w=2u l=180n
CT1366 t1366 0 0.1f
M3563 t1363 ni15 t1366 0 nch w=1u l=180n
M3564 t1366 t1362 0 0 nch w=1u l=180n
M3565 t1364 nw149 vdd vdd pch w=2u l=180n
M3566 t1364 t1362 vdd vdd pch w=2u l=180n
CT1367 t1367 0 0.1f
M3567 t1364 nw149 t1367 0 nch w=1u l=180n
M3568 t1367 t1362 0 0 nch w=1u l=180n
M3569 nw418 t1363 vdd vdd pch w=2u l=180n
M3570 nw418 t1364 vdd vdd pch w=2u l=180n
CT1368 t1368 0 0.1f
M3571 nw418 t1363 t1368 0 nch w=1u l=180n
M3572 t1368 t1364 0 0 nch w=1u l=180n
Cnw418 nw418 0 2f
M3573 nw419 nw150 vdd vdd pch w=2u l=180n
M3574 nw419 nw152 vdd vdd pch w=2u l=180n
CT1369 t1369 0 0.1f
M3575 nw419 nw150 t1369 0 nch w=1u l=180n
M3576 t1369 nw152 0 0 nch w=1u l=180n
Cnw419 nw419 0 2f
M3577 nw420 nw152 0 0 nch w=1u l=180n
M3578 nw420 nw155 0 0 nch w=1u l=180n
CT1370 t1370 0 0.1f
M3579 t1370 nw152 vdd vdd pch w=2u l=180n
M3580 nw420 nw155 t1370 vdd pch w=2u l=180n
Cnw420 nw420 0 2f
CT1371 t1371 0 0.1f
M3581 t1371 nw154 vdd vdd pch w=2u l=180n
M3582 t1371 nw158 vdd vdd pch w=2u l=180n
CT1372 t1372 0 0.1f
M3583 t1371 nw154 t1372 0 nch w=1u l=180n
M3584 t1372 nw158 0 0 nch w=1u l=180n
M3585 nw421 t1371 vdd vdd pch w=2u l=180n
M3586 nw421 t1371 0 0 nch w=1u l=180n
Cnw421 nw421 0 2f
CT1373 t1373 0 0.1f
M3587 t1373 nw156 0 0 nch w=1u l=180n
M3588 t1373 nw161 0 0 nch w=1u l=180n
CT1374 t1374 0 0.1f
M3589 t1374 nw156 vdd vdd pch w=2u l=180n
M3590 t1373 nw161 t1374 vdd pch w=2u l=180n
M3591 nw422 t1373 vdd vdd pch w=2u l=180n
M3592 nw422 t1373 0 0 nch w=1u l=180n
Cnw422 nw422 0 2f
CT1375 t1375 0 0.1f
CT1376 t1376 0 0.1f
CT1377 t1377 0 0.1f
M3593 t1375 nw158 vdd vdd pch w=2u l=180n
M3594 t1375 nw164 vdd vdd pch w=2u l=180n
CT1378 t1378 0 0.1f
M3595 t1375 nw158 t1378 0 nch w=1u l=180n
M3596 t1378 nw164 0 0 nch w=1u l=180n
M3597 t1376 nw158 vdd vdd pch w=2u l=180n
M3598 t1376 t1375 vdd vdd pch w=2u l=180n
CT1379 t1379 0 0.1f
M3599 t1376 nw158 t1379 0 nch w=1u l=180n
M3600 t1379 t1375 0 0 nch w=1u l=180n
M3601 t1377 nw164 vdd vdd pch w=2u l=180n
M3602 t1377 t1375 vdd vdd pch w=2u l=180n
CT1380 t1380 0 0.1f
M3603 t1377 nw164 t1380 0 nch w=1u l=180n
M3604 t1380 t1375 0 0 nch w=1u l=180n
M3605 nw423 t1376 vdd vdd pch w=2u l=180n
M3606 nw423 t1377 vdd vdd pch w=2u l=180n
CT1381 t1381 0 0.1f
M3607 nw423 t1376 t1381 0 nch w=1u l=180n
M3608 t1381 t1377 0 0 nch w=1u l=180n
Cnw423 nw423 0 2f
M3609 nw424 nw160 vdd vdd pch w=2u l=180n
M3610 nw424 nw167 vdd vdd pch w=2u l=180n
CT1382 t1382 0 0.1f
M3611 nw424 nw160 t1382 0 nch w=1u l=180n
M3612 t1382 nw167 0 0 nch w=1u l=180n
Cnw424 nw424 0 2f
M3613 nw425 nw162 0 0 nch w=1u l=180n
M3614 nw425 nw170 0 0 nch w=1u l=180n
CT1383 t1383 0 0.1f
M3615 t1383 nw162 vdd vdd pch w=2u l=180n
M3616 nw425 nw170 t1383 vdd pch w=2u l=180n
Cnw425 nw425 0 2f
CT1384 t1384 0 0.1f
M3617 t1384 nw164 vdd vdd pch w=2u l=180n
M3618 t1384 nw173 vdd vdd pch w=2u l=180n
CT1385 t1385 0 0.1f
M3619 t1384 nw164 t1385 0 nch w=1u l=180n
M3620 t1385 nw173 0 0 nch w=1u l=180n
M3621 nw426 t1384 vdd vdd pch w=2u l=180n
M3622 nw426 t1384 0 0 nch w=1u l=180n
Cnw426 nw426 0 2f
CT1386 t1386 0 0.1f
M3623 t1386 nw166 0 0 nch w=1u l=180n
M3624 t1386 nw176 0 0 nch w=1u l=180n
CT1387 t1387 0 0.1f
M3625 t1387 nw166 vdd vdd pch w=2u l=180n
M3626 t1386 nw176 t1387 vdd pch w=2u l=180n
M3627 nw427 t1386 vdd vdd pch w=2u l=180n
M3628 nw427 t1386 0 0 nch w=1u l=180n
Cnw427 nw427 0 2f
CT1388 t1388 0 0.1f
CT1389 t1389 0 0.1f
CT1390 t1390 0 0.1f
M3629 t1388 nw168 vdd vdd pch w=2u l=180n
M3630 t1388 nw179 vdd vdd pch w=2u l=180n
CT1391 t1391 0 0.1f
M3631 t1388 nw168 t1391 0 nch w=1u l=180n
M3632 t1391 nw179 0 0 nch w=1u l=180n
M3633 t1389 nw168 vdd vdd pch w=2u l=180n
M3634 t1389 t1388 vdd vdd pch w=2u l=180n
CT1392 t1392 0 0.1f
M3635 t1389 nw168 t1392 0 nch w=1u l=180n
M3636 t1392 t1388 0 0 nch w=1u l=180n
M3637 t1390 nw179 vdd vdd pch w=2u l=180n
M3638 t1390 t1388 vdd vdd pch w=2u l=180n
CT1393 t1393 0 0.1f
M3639 t1390 nw179 t1393 0 nch w=1u l=180n
M3640 t1393 t1388 0 0 nch w=1u l=180n
M3641 nw428 t1389 vdd vdd pch w=2u l=180n
M3642 nw428 t1390 vdd vdd pch w=2u l=180n
CT1394 t1394 0 0.1f
M3643 nw428 t1389 t1394 0 nch w=1u l=180n
M3644 t1394 t1390 0 0 nch w=1u l=180n
Cnw428 nw428 0 2f
M3645 nw429 nw170 vdd vdd pch w=2u l=180n
M3646 nw429 nw182 vdd vdd pch w=2u l=180n
CT1395 t1395 0 0.1f
M3647 nw429 nw170 t1395 0 nch w=1u l=180n
M3648 t1395 nw182 0 0 nch w=1u l=180n
Cnw429 nw429 0 2f
M3649 nw430 nw172 0 0 nch w=1u l=180n
M3650 nw430 nw185 0 0 nch w=1u l=180n
CT1396 t1396 0 0.1f
M3651 t1396 nw172 vdd vdd pch w=2u l=180n
M3652 nw430 nw185 t1396 vdd pch w=2u l=180n
Cnw430 nw430 0 2f
CT1397 t1397 0 0.1f
M3653 t1397 nw174 vdd vdd pch w=2u l=180n
M3654 t1397 nw188 vdd vdd pch w=2u l=180n
CT1398 t1398 0 0.1f
M3655 t1397 nw174 t1398 0 nch w=1u l=180n
M3656 t1398 nw188 0 0 nch w=1u l=180n
M3657 nw431 t1397 vdd vdd pch w=2u l=180n
M3658 nw431 t1397 0 0 nch w=1u l=180n
Cnw431 nw431 0 2f
CT1399 t1399 0 0.1f
M3659 t1399 nw176 0 0 nch w=1u l=180n
M3660 t1399 nw191 0 0 nch w=1u l=180n
CT1400 t1400 0 0.1f
M3661 t1400 nw176 vdd vdd pch w=2u l=180n
M3662 t1399 nw191 t1400 vdd pch w=2u l=180n
M3663 nw432 t1399 vdd vdd pch w=2u l=180n
M3664 nw432 t1399 0 0 nch w=1u l=180n
Cnw432 nw432 0 2f
CT1401 t1401 0 0.1f
CT1402 t1402 0 0.1f
CT1403 t1403 0 0.1f
M3665 t1401 nw178 vdd vdd pch w=2u l=180n
M3666 t1401 nw194 vdd vdd pch w=2u l=180n
CT1404 t1404 0 0.1f
M3667 t1401 nw178 t1404 0 nch w=1u l=180n
M3668 t1404 nw194 0 0 nch w=1u l=180n
M3669 t1402 nw178 vdd vdd pch w=2u l=180n
M3670 t1402 t1401 vdd vdd pch w=2u l=180n
CT1405 t1405 0 0.1f
M3671 t1402 nw178 t1405 0 nch w=1u l=180n
M3672 t1405 t1401 0 0 nch w=1u l=180n
M3673 t1403 nw194 vdd vdd pch w=2u l=180n
M3674 t1403 t1401 vdd vdd pch w=2u l=180n
CT1406 t1406 0 0.1f
M3675 t1403 nw194 t1406 0 nch w=1u l=180n
M3676 t1406 t1401 0 0 nch w=1u l=180n
M3677 nw433 t1402 vdd vdd pch w=2u l=180n
M3678 nw433 t1403 vdd vdd pch w=2u l=180n
CT1407 t1407 0 0.1f
M3679 nw433 t1402 t1407 0 nch w=1u l=180n
M3680 t1407 t1403 0 0 nch w=1u l=180n
Cnw433 nw433 0 2f
M3681 nw434 nw180 vdd vdd pch w=2u l=180n
M3682 nw434 nw197 vdd vdd pch w=2u l=180n
CT1408 t1408 0 0.1f
M3683 nw434 nw180 t1408 0 nch w=1u l=180n
M3684 t1408 nw197 0 0 nch w=1u l=180n
Cnw434 nw434 0 2f
M3685 nw435 nw182 0 0 nch w=1u l=180n
M3686 nw435 nw200 0 0 nch w=1u l=180n
CT1409 t1409 0 0.1f
M3687 t1409 nw182 vdd vdd pch w=2u l=180n
M3688 nw435 nw200 t1409 vdd pch w=2u l=180n
Cnw435 nw435 0 2f
CT1410 t1410 0 0.1f
M3689 t1410 nw184 vdd vdd pch w=2u l=180n
M3690 t1410 nw203 vdd vdd pch w=2u l=180n
CT1411 t1411 0 0.1f
M3691 t1410 nw184 t1411 0 nch w=1u l=180n
M3692 t1411 nw203 0 0 nch w=1u l=180n
M3693 nw436 t1410 vdd vdd pch w=2u l=180n
M3694 nw436 t1410 0 0 nch w=1u l=180n
Cnw436 nw436 0 2f
CT1412 t1412 0 0.1f
M3695 t1412 nw186 0 0 nch w=1u l=180n
M3696 t1412 nw206 0 0 nch w=1u l=180n
CT1413 t1413 0 0.1f
M3697 t1413 nw186 vdd vdd pch w=2u l=180n
M3698 t1412 nw206 t1413 vdd pch w=2u l=180n
M3699 nw437 t1412 vdd vdd pch w=2u l=180n
M3700 nw437 t1412 0 0 nch w=1u l=180n
Cnw437 nw437 0 2f
CT1414 t1414 0 0.1f
CT1415 t1415 0 0.1f
CT1416 t1416 0 0.1f
M3701 t1414 nw188 vdd vdd pch w=2u l=180n
M3702 t1414 nw209 vdd vdd pch w=2u l=180n
CT1417 t1417 0 0.1f
M3703 t1414 nw188 t1417 0 nch w=1u l=180n
M3704 t1417 nw209 0 0 nch w=1u l=180n
M3705 t1415 nw188 vdd vdd pch w=2u l=180n
M3706 t1415 t1414 vdd vdd pch w=2u l=180n
CT1418 t1418 0 0.1f
M3707 t1415 nw188 t1418 0 nch w=1u l=180n
M3708 t1418 t1414 0 0 nch w=1u l=180n
M3709 t1416 nw209 vdd vdd pch w=2u l=180n
M3710 t1416 t1414 vdd vdd pch w=2u l=180n
CT1419 t1419 0 0.1f
M3711 t1416 nw209 t1419 0 nch w=1u l=180n
M3712 t1419 t1414 0 0 nch w=1u l=180n
M3713 nw438 t1415 vdd vdd pch w=2u l=180n
M3714 nw438 t1416 vdd vdd pch w=2u l=180n
CT1420 t1420 0 0.1f
M3715 nw438 t1415 t1420 0 nch w=1u l=180n
M3716 t1420 t1416 0 0 nch w=1u l=180n
Cnw438 nw438 0 2f
M3717 nw439 nw190 vdd vdd pch w=2u l=180n
M3718 nw439 nw212 vdd vdd pch w=2u l=180n
CT1421 t1421 0 0.1f
M3719 nw439 nw190 t1421 0 nch w=1u l=180n
M3720 t1421 nw212 0 0 nch w=1u l=180n
Cnw439 nw439 0 2f
M3721 nw440 nw192 0 0 nch w=1u l=180n
M3722 nw440 nw215 0 0 nch w=1u l=180n
CT1422 t1422 0 0.1f
M3723 t1422 nw192 vdd vdd pch w=2u l=180n
M3724 nw440 nw215 t1422 vdd pch w=2u l=180n
Cnw440 nw440 0 2f
CT1423 t1423 0 0.1f
M3725 t1423 nw194 vdd vdd pch w=2u l=180n
M3726 t1423 nw218 vdd vdd pch w=2u l=180n
CT1424 t1424 0 0.1f
M3727 t1423 nw194 t1424 0 nch w=1u l=180n
M3728 t1424 nw218 0 0 nch w=1u l=180n
M3729 nw441 t1423 vdd vdd pch w=2u l=180n
M3730 nw441 t1423 0 0 nch w=1u l=180n
Cnw441 nw441 0 2f
CT1425 t1425 0 0.1f
M3731 t1425 nw196 0 0 nch w=1u l=180n
M3732 t1425 nw221 0 0 nch w=1u l=180n
CT1426 t1426 0 0.1f
M3733 t1426 nw196 vdd vdd pch w=2u l=180n
M3734 t1425 nw221 t1426 vdd pch w=2u l=180n
M3735 nw442 t1425 vdd vdd pch w=2u l=180n
M3736 nw442 t1425 0 0 nch w=1u l=180n
Cnw442 nw442 0 2f
CT1427 t1427 0 0.1f
CT1428 t1428 0 0.1f
CT1429 t1429 0 0.1f
M3737 t1427 nw198 vdd vdd pch w=2u l=180n
M3738 t1427 nw224 vdd vdd pch w=2u l=180n
CT1430 t1430 0 0.1f
M3739 t1427 nw198 t1430 0 nch w=1u l=180n
M3740 t1430 nw224 0 0 nch w=1u l=180n
M3741 t1428 nw198 vdd vdd pch w=2u l=180n
M3742 t1428 t1427 vdd vdd pch w=2u l=180n
CT1431 t1431 0 0.1f
M3743 t1428 nw198 t1431 0 nch w=1u l=180n
M3744 t1431 t1427 0 0 nch w=1u l=180n
M3745 t1429 nw224 vdd vdd pch w=2u l=180n
M3746 t1429 t1427 vdd vdd pch w=2u l=180n
CT1432 t1432 0 0.1f
M3747 t1429 nw224 t1432 0 nch w=1u l=180n
M3748 t1432 t1427 0 0 nch w=1u l=180n
M3749 nw443 t1428 vdd vdd pch w=2u l=180n
M3750 nw443 t1429 vdd vdd pch w=2u l=180n
CT1433 t1433 0 0.1f
M3751 nw443 t1428 t1433 0 nch w=1u l=180n
M3752 t1433 t1429 0 0 nch w=1u l=180n
Cnw443 nw443 0 2f
M3753 nw444 nw200 vdd vdd pch w=2u l=180n
M3754 nw444 nw227 vdd vdd pch w=2u l=180n
CT1434 t1434 0 0.1f
M3755 nw444 nw200 t1434 0 nch w=1u l=180n
M3756 t1434 nw227 0 0 nch w=1u l=180n
Cnw444 nw444 0 2f
M3757 nw445 nw202 0 0 nch w=1u l=180n
M3758 nw445 nw230 0 0 nch w=1u l=180n
CT1435 t1435 0 0.1f
M3759 t1435 nw202 vdd vdd pch w=2u l=180n
M3760 nw445 nw230 t1435 vdd pch w=2u l=180n
Cnw445 nw445 0 2f
CT1436 t1436 0 0.1f
M3761 t1436 nw204 vdd vdd pch w=2u l=180n
M3762 t1436 nw233 vdd vdd pch w=2u l=180n
CT1437 t1437 0 0.1f
M3763 t1436 nw204 t1437 0 nch w=1u l=180n
M3764 t1437 nw233 0 0 nch w=1u l=180n
M3765 nw446 t1436 vdd vdd pch w=2u l=180n
M3766 nw446 t1436 0 0 nch w=1u l=180n
Cnw446 nw446 0 2f
CT1438 t1438 0 0.1f
M3767 t1438 nw206 0 0 nch w=1u l=180n
M3768 t1438 nw236 0 0 nch w=1u l=180n
CT1439 t1439 0 0.1f
M3769 t1439 nw206 vdd vdd pch w=2u l=180n
M3770 t1438 nw236 t1439 vdd pch w=2u l=180n
M3771 nw447 t1438 vdd vdd pch w=2u l=180n
M3772 nw447 t1438 0 0 nch w=1u l=180n
Cnw447 nw447 0 2f
CT1440 t1440 0 0.1f
CT1441 t1441 0 0.1f
CT1442 t1442 0 0.1f
M3773 t1440 nw208 vdd vdd pch w=2u l=180n
M3774 t1440 nw239 vdd vdd pch w=2u l=180n
CT1443 t1443 0 0.1f
M3775 t1440 nw208 t1443 0 nch w=1u l=180n
M3776 t1443 nw239 0 0 nch w=1u l=180n
M3777 t1441 nw208 vdd vdd pch w=2u l=180n
M3778 t1441 t1440 vdd vdd pch w=2u l=180n
CT1444 t1444 0 0.1f
M3779 t1441 nw208 t1444 0 nch w=1u l=180n
M3780 t1444 t1440 0 0 nch w=1u l=180n
M3781 t1442 nw239 vdd vdd pch w=2u l=180n
M3782 t1442 t1440 vdd vdd pch w=2u l=180n
CT1445 t1445 0 0.1f
M3783 t1442 nw239 t1445 0 nch w=1u l=180n
M3784 t1445 t1440 0 0 nch w=1u l=180n
M3785 nw448 t1441 vdd vdd pch w=2u l=180n
M3786 nw448 t1442 vdd vdd pch w=2u l=180n
CT1446 t1446 0 0.1f
M3787 nw448 t1441 t1446 0 nch w=1u l=180n
M3788 t1446 t1442 0 0 nch w=1u l=180n
Cnw448 nw448 0 2f
M3789 nw449 nw210 vdd vdd pch w=2u l=180n
M3790 nw449 nw242 vdd vdd pch w=2u l=180n
CT1447 t1447 0 0.1f
M3791 nw449 nw210 t1447 0 nch w=1u l=180n
M3792 t1447 nw242 0 0 nch w=1u l=180n
Cnw449 nw449 0 2f
M3793 nw450 nw212 0 0 nch w=1u l=180n
M3794 nw450 nw245 0 0 nch w=1u l=180n
CT1448 t1448 0 0.1f
M3795 t1448 nw212 vdd vdd pch w=2u l=180n
M3796 nw450 nw245 t1448 vdd pch w=2u l=180n
Cnw450 nw450 0 2f
CT1449 t1449 0 0.1f
M3797 t1449 nw214 vdd vdd pch w=2u l=180n
M3798 t1449 nw248 vdd vdd pch w=2u l=180n
CT1450 t1450 0 0.1f
M3799 t1449 nw214 t1450 0 nch w=1u l=180n
M3800 t1450 nw248 0 0 nch w=1u l=180n
M3801 nw451 t1449 vdd vdd pch w=2u l=180n
M3802 nw451 t1449 0 0 nch w=1u l=180n
Cnw451 nw451 0 2f
CT1451 t1451 0 0.1f
M3803 t1451 nw216 0 0 nch w=1u l=180n
M3804 t1451 nw251 0 0 nch w=1u l=180n
CT1452 t1452 0 0.1f
M3805 t1452 nw216 vdd vdd pch w=2u l=180n
M3806 t1451 nw251 t1452 vdd pch w=2u l=180n
M3807 nw452 t1451 vdd vdd pch w=2u l=180n
M3808 nw452 t1451 0 0 nch w=1u l=180n
Cnw452 nw452 0 2f
CT1453 t1453 0 0.1f
CT1454 t1454 0 0.1f
CT1455 t1455 0 0.1f
M3809 t1453 nw218 vdd vdd pch w=2u l=180n
M3810 t1453 nw254 vdd vdd pch w=2u l=180n
CT1456 t1456 0 0.1f
M3811 t1453 nw218 t1456 0 nch w=1u l=180n
M3812 t1456 nw254 0 0 nch w=1u l=180n
M3813 t1454 nw218 vdd vdd pch w=2u l=180n
M3814 t1454 t1453 vdd vdd pch w=2u l=180n
CT1457 t1457 0 0.1f
M3815 t1454 nw218 t1457 0 nch w=1u l=180n
M3816 t1457 t1453 0 0 nch w=1u l=180n
M3817 t1455 nw254 vdd vdd pch w=2u l=180n
M3818 t1455 t1453 vdd vdd pch w=2u l=180n
CT1458 t1458 0 0.1f
M3819 t1455 nw254 t1458 0 nch w=1u l=180n
M3820 t1458 t1453 0 0 nch w=1u l=180n
M3821 nw453 t1454 vdd vdd pch w=2u l=180n
M3822 nw453 t1455 vdd vdd pch w=2u l=180n
CT1459 t1459 0 0.1f
M3823 nw453 t1454 t1459 0 nch w=1u l=180n
M3824 t1459 t1455 0 0 nch w=1u l=180n
Cnw453 nw453 0 2f
M3825 nw454 nw220 vdd vdd pch w=2u l=180n
M3826 nw454 nw257 vdd vdd pch w=2u l=180n
CT1460 t1460 0 0.1f
M3827 nw454 nw220 t1460 0 nch w=1u l=180n
M3828 t1460 nw257 0 0 nch w=1u l=180n
Cnw454 nw454 0 2f
M3829 nw455 nw222 0 0 nch w=1u l=180n
M3830 nw455 nw260 0 0 nch w=1u l=180n
CT1461 t1461 0 0.1f
M3831 t1461 nw222 vdd vdd pch w=2u l=180n
M3832 nw455 nw260 t1461 vdd pch w=2u l=180n
Cnw455 nw455 0 2f
CT1462 t1462 0 0.1f
M3833 t1462 nw224 vdd vdd pch w=2u l=180n
M3834 t1462 nw263 vdd vdd pch w=2u l=180n
CT1463 t1463 0 0.1f
M3835 t1462 nw224 t1463 0 nch w=1u l=180n
M3836 t1463 nw263 0 0 nch w=1u l=180n
M3837 nw456 t1462 vdd vdd pch w=2u l=180n
M3838 nw456 t1462 0 0 nch w=1u l=180n
Cnw456 nw456 0 2f
CT1464 t1464 0 0.1f
M3839 t1464 nw226 0 0 nch w=1u l=180n
M3840 t1464 nw266 0 0 nch w=1u l=180n
CT1465 t1465 0 0.1f
M3841 t1465 nw226 vdd vdd pch w=2u l=180n
M3842 t1464 nw266 t1465 vdd pch w=2u l=180n
M3843 nw457 t1464 vdd vdd pch w=2u l=180n
M3844 nw457 t1464 0 0 nch w=1u l=180n
Cnw457 nw457 0 2f
CT1466 t1466 0 0.1f
CT1467 t1467 0 0.1f
CT1468 t1468 0 0.1f
M3845 t1466 nw228 vdd vdd pch w=2u l=180n
M3846 t1466 nw269 vdd vdd pch w=2u l=180n
CT1469 t1469 0 0.1f
M3847 t1466 nw228 t1469 0 nch w=1u l=180n
M3848 t1469 nw269 0 0 nch w=1u l=180n
M3849 t1467 nw228 vdd vdd pch w=2u l=180n
M3850 t1467 t1466 vdd vdd pch w=2u l=180n
CT1470 t1470 0 0.1f
M3851 t1467 nw228 t1470 0 nch w=1u l=180n
M3852 t1470 t1466 0 0 nch w=1u l=180n
M3853 t1468 nw269 vdd vdd pch w=2u l=180n
M3854 t1468 t1466 vdd vdd pch w=2u l=180n
CT1471 t1471 0 0.1f
M3855 t1468 nw269 t1471 0 nch w=1u l=180n
M3856 t1471 t1466 0 0 nch w=1u l=180n
M3857 nw458 t1467 vdd vdd pch w=2u l=180n
M3858 nw458 t1468 vdd vdd pch w=2u l=180n
CT1472 t1472 0 0.1f
M3859 nw458 t1467 t1472 0 nch w=1u l=180n
M3860 t1472 t1468 0 0 nch w=1u l=180n
Cnw458 nw458 0 2f
M3861 nw459 nw230 vdd vdd pch w=2u l=180n
M3862 nw459 nw272 vdd vdd pch w=2u l=180n
CT1473 t1473 0 0.1f
M3863 nw459 nw230 t1473 0 nch w=1u l=180n
M3864 t1473 nw272 0 0 nch w=1u l=180n
Cnw459 nw459 0 2f
M3865 nw460 nw232 0 0 nch w=1u l=180n
M3866 nw460 nw275 0 0 nch w=1u l=180n
CT1474 t1474 0 0.1f
M3867 t1474 nw232 vdd vdd pch w=2u l=180n
M3868 nw460 nw275 t1474 vdd pch w=2u l=180n
Cnw460 nw460 0 2f
CT1475 t1475 0 0.1f
M3869 t1475 nw234 vdd vdd pch w=2u l=180n
M3870 t1475 nw278 vdd vdd pch w=2u l=180n
CT1476 t1476 0 0.1f
M3871 t1475 nw234 t1476 0 nch w=1u l=180n
M3872 t1476 nw278 0 0 nch w=1u l=180n
M3873 nw461 t1475 vdd vdd pch w=2u l=180n
M3874 nw461 t1475 0 0 nch w=1u l=180n
Cnw461 nw461 0 2f
CT1477 t1477 0 0.1f
M3875 t1477 nw236 0 0 nch w=1u l=180n
M3876 t1477 nw281 0 0 nch w=1u l=180n
CT1478 t1478 0 0.1f
M3877 t1478 nw236 vdd vdd pch w=2u l=180n
M3878 t1477 nw281 t1478 vdd pch w=2u l=180n
M3879 nw462 t1477 vdd vdd pch w=2u l=180n
M3880 nw462 t1477 0 0 nch w=1u l=180n
Cnw462 nw462 0 2f
CT1479 t1479 0 0.1f
CT1480 t1480 0 0.1f
CT1481 t1481 0 0.1f
M3881 t1479 nw238 vdd vdd pch w=2u l=180n
M3882 t1479 nw284 vdd vdd pch w=2u l=180n
CT1482 t1482 0 0.1f
M3883 t1479 nw238 t1482 0 nch w=1u l=180n
M3884 t1482 nw284 0 0 nch w=1u l=180n
M3885 t1480 nw238 vdd vdd pch w=2u l=180n
M3886 t1480 t1479 vdd vdd pch w=2u l=180n
CT1483 t1483 0 0.1f
M3887 t1480 nw238 t1483 0 nch w=1u l=180n
M3888 t1483 t1479 0 0 nch w=1u l=180n
M3889 t1481 nw284 vdd vdd pch w=2u l=180n
M3890 t1481 t1479 vdd vdd pch w=2u l=180n
CT1484 t1484 0 0.1f
M3891 t1481 nw284 t1484 0 nch w=1u l=180n
M3892 t1484 t1479 0 0 nch w=1u l=180n
M3893 nw463 t1480 vdd vdd pch w=2u l=180n
M3894 nw463 t1481 vdd vdd pch w=2u l=180n
CT1485 t1485 0 0.1f
M3895 nw463 t1480 t1485 0 nch w=1u l=180n
M3896 t1485 t1481 0 0 nch w=1u l=180n
Cnw463 nw463 0 2f
M3897 nw464 nw240 vdd vdd pch w=2u l=180n
M3898 nw464 nw287 vdd vdd pch w=2u l=180n
CT1486 t1486 0 0.1f
M3899 nw464 nw240 t1486 0 nch w=1u l=180n
M3900 t1486 nw287 0 0 nch w=1u l=180n
Cnw464 nw464 0 2f
M3901 nw465 nw242 0 0 nch w=1u l=180n
M3902 nw465 nw290 0 0 nch w=1u l=180n
CT1487 t1487 0 0.1f
M3903 t1487 nw242 vdd vdd pch w=2u l=180n
M3904 nw465 nw290 t1487 vdd pch w=2u l=180n
Cnw465 nw465 0 2f
CT1488 t1488 0 0.1f
M3905 t1488 nw244 vdd vdd pch w=2u l=180n
M3906 t1488 nw293 vdd vdd pch w=2u l=180n
CT1489 t1489 0 0.1f
M3907 t1488 nw244 t1489 0 nch w=1u l=180n
M3908 t1489 nw293 0 0 nch w=1u l=180n
M3909 nw466 t1488 vdd vdd pch w=2u l=180n
M3910 nw466 t1488 0 0 nch w=1u l=180n
Cnw466 nw466 0 2f
CT1490 t1490 0 0.1f
M3911 t1490 nw246 0 0 nch w=1u l=180n
M3912 t1490 nw296 0 0 nch w=1u l=180n
CT1491 t1491 0 0.1f
M3913 t1491 nw246 vdd vdd pch w=2u l=180n
M3914 t1490 nw296 t1491 vdd pch w=2u l=180n
M3915 nw467 t1490 vdd vdd pch w=2u l=180n
M3916 nw467 t1490 0 0 nch w=1u l=180n
Cnw467 nw467 0 2f
CT1492 t1492 0 0.1f
CT1493 t1493 0 0.1f
CT1494 t1494 0 0.1f
M3917 t1492 nw248 vdd vdd pch w=2u l=180n
M3918 t1492 nw299 vdd vdd pch w=2u l=180n
CT1495 t1495 0 0.1f
M3919 t1492 nw248 t1495 0 nch w=1u l=180n
M3920 t1495 nw299 0 0 nch w=1u l=180n
M3921 t1493 nw248 vdd vdd pch w=2u l=180n
M3922 t1493 t1492 vdd vdd pch w=2u l=180n
CT1496 t1496 0 0.1f
M3923 t1493 nw248 t1496 0 nch w=1u l=180n
M3924 t1496 t1492 0 0 nch w=1u l=180n
M3925 t1494 nw299 vdd vdd pch w=2u l=180n
M3926 t1494 t1492 vdd vdd pch w=2u l=180n
CT1497 t1497 0 0.1f
M3927 t1494 nw299 t1497 0 nch w=1u l=180n
M3928 t1497 t1492 0 0 nch w=1u l=180n
M3929 nw468 t1493 vdd vdd pch w=2u l=180n
M3930 nw468 t1494 vdd vdd pch w=2u l=180n
CT1498 t1498 0 0.1f
M3931 nw468 t1493 t1498 0 nch w=1u l=180n
M3932 t1498 t1494 0 0 nch w=1u l=180n
Cnw468 nw468 0 2f
M3933 nw469 nw250 vdd vdd pch w=2u l=180n
M3934 nw469 nw302 vdd vdd pch w=2u l=180n
CT1499 t1499 0 0.1f
M3935 nw469 nw250 t1499 0 nch w=1u l=180n
M3936 t1499 nw302 0 0 nch w=1u l=180n
Cnw469 nw469 0 2f
M3937 nw470 nw252 0 0 nch w=1u l=180n
M3938 nw470 nw305 0 0 nch w=1u l=180n
CT1500 t1500 0 0.1f
M3939 t1500 nw252 vdd vdd pch w=2u l=180n
M3940 nw470 nw305 t1500 vdd pch w=2u l=180n
Cnw470 nw470 0 2f
CT1501 t1501 0 0.1f
M3941 t1501 nw254 vdd vdd pch w=2u l=180n
M3942 t1501 nw308 vdd vdd pch w=2u l=180n
CT1502 t1502 0 0.1f
M3943 t1501 nw254 t1502 0 nch w=1u l=180n
M3944 t1502 nw308 0 0 nch w=1u l=180n
M3945 nw471 t1501 vdd vdd pch w=2u l=180n
M3946 nw471 t1501 0 0 nch w=1u l=180n
Cnw471 nw471 0 2f
CT1503 t1503 0 0.1f
M3947 t1503 nw256 0 0 nch w=1u l=180n
M3948 t1503 nw311 0 0 nch w=1u l=180n
CT1504 t1504 0 0.1f
M3949 t1504 nw256 vdd vdd pch w=2u l=180n
M3950 t1503 nw311 t1504 vdd pch w=2u l=180n
M3951 nw472 t1503 vdd vdd pch w=2u l=180n
M3952 nw472 t1503 0 0 nch w=1u l=180n
Cnw472 nw472 0 2f
CT1505 t1505 0 0.1f
CT1506 t1506 0 0.1f
CT1507 t1507 0 0.1f
M3953 t1505 nw258 vdd vdd pch w=2u l=180n
M3954 t1505 nw314 vdd vdd pch w=2u l=180n
CT1508 t1508 0 0.1f
M3955 t1505 nw258 t1508 0 nch w=1u l=180n
M3956 t1508 nw314 0 0 nch w=1u l=180n
M3957 t1506 nw258 vdd vdd pch w=2u l=180n
M3958 t1506 t1505 vdd vdd pch w=2u l=180n
CT1509 t1509 0 0.1f
M3959 t1506 nw258 t1509 0 nch w=1u l=180n
M3960 t1509 t1505 0 0 nch w=1u l=180n
M3961 t1507 nw314 vdd vdd pch w=2u l=180n
M3962 t1507 t1505 vdd vdd pch w=2u l=180n
CT1510 t1510 0 0.1f
M3963 t1507 nw314 t1510 0 nch w=1u l=180n
M3964 t1510 t1505 0 0 nch w=1u l=180n
M3965 nw473 t1506 vdd vdd pch w=2u l=180n
M3966 nw473 t1507 vdd vdd pch w=2u l=180n
CT1511 t1511 0 0.1f
M3967 nw473 t1506 t1511 0 nch w=1u l=180n
M3968 t1511 t1507 0 0 nch w=1u l=180n
Cnw473 nw473 0 2f
M3969 nw474 nw260 vdd vdd pch w=2u l=180n
M3970 nw474 nw317 vdd vdd pch w=2u l=180n
CT1512 t1512 0 0.1f
M3971 nw474 nw260 t1512 0 nch w=1u l=180n
M3972 t1512 nw317 0 0 nch w=1u l=180n
Cnw474 nw474 0 2f
M3973 nw475 nw262 0 0 nch w=1u l=180n
M3974 nw475 nw320 0 0 nch w=1u l=180n
CT1513 t1513 0 0.1f
M3975 t1513 nw262 vdd vdd pch w=2u l=180n
M3976 nw475 nw320 t1513 vdd pch w=2u l=180n
Cnw475 nw475 0 2f
CT1514 t1514 0 0.1f
M3977 t1514 nw264 vdd vdd pch w=2u l=180n
M3978 t1514 nw323 vdd vdd pch w=2u l=180n
CT1515 t1515 0 0.1f
M3979 t1514 nw264 t1515 0 nch w=1u l=180n
M3980 t1515 nw323 0 0 nch w=1u l=180n
M3981 nw476 t1514 vdd vdd pch w=2u l=180n
M3982 nw476 t1514 0 0 nch w=1u l=180n
Cnw476 nw476 0 2f
CT1516 t1516 0 0.1f
M3983 t1516 nw266 0 0 nch w=1u l=180n
M3984 t1516 nw326 0 0 nch w=1u l=180n
CT1517 t1517 0 0.1f
M3985 t1517 nw266 vdd vdd pch w=2u l=180n
M3986 t1516 nw326 t1517 vdd pch w=2u l=180n
M3987 nw477 t1516 vdd vdd pch w=2u l=180n
M3988 nw477 t1516 0 0 nch w=1u l=180n
Cnw477 nw477 0 2f
CT1518 t1518 0 0.1f
CT1519 t1519 0 0.1f
CT1520 t1520 0 0.1f
M3989 t1518 nw268 vdd vdd pch w=2u l=180n
M3990 t1518 nw329 vdd vdd pch w=2u l=180n
CT1521 t1521 0 0.1f
M3991 t1518 nw268 t1521 0 nch w=1u l=180n
M3992 t1521 nw329 0 0 nch w=1u l=180n
M3993 t1519 nw268 vdd vdd pch w=2u l=180n
M3994 t1519 t1518 vdd vdd pch w=2u l=180n
CT1522 t1522 0 0.1f
M3995 t1519 nw268 t1522 0 nch w=1u l=180n
M3996 t1522 t1518 0 0 nch w=1u l=180n
M3997 t1520 nw329 vdd vdd pch w=2u l=180n
M3998 t1520 t1518 vdd vdd pch w=2u l=180n
CT1523 t1523 0 0.1f
M3999 t1520 nw329 t1523 0 nch w=1u l=180n
M4000 t1523 t1518 0 0 nch w=1u l=180n
M4001 nw478 t1519 vdd vdd pch w=2u l=180n
M4002 nw478 t1520 vdd vdd pch w=2u l=180n
CT1524 t1524 0 0.1f
M4003 nw478 t1519 t1524 0 nch w=1u l=180n
M4004 t1524 t1520 0 0 nch w=1u l=180n
Cnw478 nw478 0 2f
M4005 nw479 nw270 vdd vdd pch w=2u l=180n
M4006 nw479 nw332 vdd vdd pch w=2u l=180n
CT1525 t1525 0 0.1f
M4007 nw479 nw270 t1525 0 nch w=1u l=180n
M4008 t1525 nw332 0 0 nch w=1u l=180n
Cnw479 nw479 0 2f
M4009 nw480 nw272 0 0 nch w=1u l=180n
M4010 nw480 nw335 0 0 nch w=1u l=180n
CT1526 t1526 0 0.1f
M4011 t1526 nw272 vdd vdd pch w=2u l=180n
M4012 nw480 nw335 t1526 vdd pch w=2u l=180n
Cnw480 nw480 0 2f
CT1527 t1527 0 0.1f
M4013 t1527 nw274 vdd vdd pch w=2u l=180n
M4014 t1527 nw338 vdd vdd pch w=2u l=180n
CT1528 t1528 0 0.1f
M4015 t1527 nw274 t1528 0 nch w=1u l=180n
M4016 t1528 nw338 0 0 nch w=1u l=180n
M4017 nw481 t1527 vdd vdd pch w=2u l=180n
M4018 nw481 t1527 0 0 nch w=1u l=180n
Cnw481 nw481 0 2f
CT1529 t1529 0 0.1f
M4019 t1529 nw276 0 0 nch w=1u l=180n
M4020 t1529 nw341 0 0 nch w=1u l=180n
CT1530 t1530 0 0.1f
M4021 t1530 nw276 vdd vdd pch w=2u l=180n
M4022 t1529 nw341 t1530 vdd pch w=2u l=180n
M4023 nw482 t1529 vdd vdd pch w=2u l=180n
M4024 nw482 t1529 0 0 nch w=1u l=180n
Cnw482 nw482 0 2f
CT1531 t1531 0 0.1f
CT1532 t1532 0 0.1f
CT1533 t1533 0 0.1f
M4025 t1531 nw278 vdd vdd pch w=2u l=180n
M4026 t1531 nw344 vdd vdd pch w=2u l=180n
CT1534 t1534 0 0.1f
M4027 t1531 nw278 t1534 0 nch w=1u l=180n
M4028 t1534 nw344 0 0 nch w=1u l=180n
M4029 t1532 nw278 vdd vdd pch w=2u l=180n
M4030 t1532 t1531 vdd vdd pch w=2u l=180n
CT1535 t1535 0 0.1f
M4031 t1532 nw278 t1535 0 nch w=1u l=180n
M4032 t1535 t1531 0 0 nch w=1u l=180n
M4033 t1533 nw344 vdd vdd pch w=2u l=180n
M4034 t1533 t1531 vdd vdd pch w=2u l=180n
CT1536 t1536 0 0.1f
M4035 t1533 nw344 t1536 0 nch w=1u l=180n
M4036 t1536 t1531 0 0 nch w=1u l=180n
M4037 nw483 t1532 vdd vdd pch w=2u l=180n
M4038 nw483 t1533 vdd vdd pch w=2u l=180n
CT1537 t1537 0 0.1f
M4039 nw483 t1532 t1537 0 nch w=1u l=180n
M4040 t1537 t1533 0 0 nch w=1u l=180n
Cnw483 nw483 0 2f
M4041 nw484 nw280 vdd vdd pch w=2u l=180n
M4042 nw484 nw347 vdd vdd pch w=2u l=180n
CT1538 t1538 0 0.1f
M4043 nw484 nw280 t1538 0 nch w=1u l=180n
M4044 t1538 nw347 0 0 nch w=1u l=180n
Cnw484 nw484 0 2f
M4045 nw485 nw282 0 0 nch w=1u l=180n
M4046 nw485 nw350 0 0 nch w=1u l=180n
CT1539 t1539 0 0.1f
M4047 t1539 nw282 vdd vdd pch w=2u l=180n
M4048 nw485 nw350 t1539 vdd pch w=2u l=180n
Cnw485 nw485 0 2f
CT1540 t1540 0 0.1f
M4049 t1540 nw284 vdd vdd pch w=2u l=180n
M4050 t1540 nw353 vdd vdd pch w=2u l=180n
CT1541 t1541 0 0.1f
M4051 t1540 nw284 t1541 0 nch w=1u l=180n
M4052 t1541 nw353 0 0 nch w=1u l=180n
M4053 nw486 t1540 vdd vdd pch w=2u l=180n
M4054 nw486 t1540 0 0 nch w=1u l=180n
Cnw486 nw486 0 2f
CT1542 t1542 0 0.1f
M4055 t1542 nw286 0 0 nch w=1u l=180n
M4056 t1542 nw356 0 0 nch w=1u l=180n
CT1543 t1543 0 0.1f
M4057 t1543 nw286 vdd vdd pch w=2u l=180n
M4058 t1542 nw356 t1543 vdd pch w=2u l=180n
M4059 nw487 t1542 vdd vdd pch w=2u l=180n
M4060 nw487 t1542 0 0 nch w=1u l=180n
Cnw487 nw487 0 2f
CT1544 t1544 0 0.1f
CT1545 t1545 0 0.1f
CT1546 t1546 0 0.1f
M4061 t1544 nw288 vdd vdd pch w=2u l=180n
M4062 t1544 nw359 vdd vdd pch w=2u l=180n
CT1547 t1547 0 0.1f
M4063 t1544 nw288 t1547 0 nch w=1u l=180n
M4064 t1547 nw359 0 0 nch w=1u l=180n
M4065 t1545 nw288 vdd vdd pch w=2u l=180n
M4066 t1545 t1544 vdd vdd pch w=2u l=180n
CT1548 t1548 0 0.1f
M4067 t1545 nw288 t1548 0 nch w=1u l=180n
M4068 t1548 t1544 0 0 nch w=1u l=180n
M4069 t1546 nw359 vdd vdd pch w=2u l=180n
M4070 t1546 t1544 vdd vdd pch w=2u l=180n
CT1549 t1549 0 0.1f
M4071 t1546 nw359 t1549 0 nch w=1u l=180n
M4072 t1549 t1544 0 0 nch w=1u l=180n
M4073 nw488 t1545 vdd vdd pch w=2u l=180n
M4074 nw488 t1546 vdd vdd pch w=2u l=180n
CT1550 t1550 0 0.1f
M4075 nw488 t1545 t1550 0 nch w=1u l=180n
M4076 t1550 t1546 0 0 nch w=1u l=180n
Cnw488 nw488 0 2f
M4077 nw489 nw290 vdd vdd pch w=2u l=180n
M4078 nw489 nw362 vdd vdd pch w=2u l=180n
CT1551 t1551 0 0.1f
M4079 nw489 nw290 t1551 0 nch w=1u l=180n
M4080 t1551 nw362 0 0 nch w=1u l=180n
Cnw489 nw489 0 2f
M4081 nw490 nw292 0 0 nch w=1u l=180n
M4082 nw490 nw365 0 0 nch w=1u l=180n
CT1552 t1552 0 0.1f
M4083 t1552 nw292 vdd vdd pch w=2u l=180n
M4084 nw490 nw365 t1552 vdd pch w=2u l=180n
Cnw490 nw490 0 2f
CT1553 t1553 0 0.1f
M4085 t1553 nw294 vdd vdd pch w=2u l=180n
M4086 t1553 nw368 vdd vdd pch w=2u l=180n
CT1554 t1554 0 0.1f
M4087 t1553 nw294 t1554 0 nch w=1u l=180n
M4088 t1554 nw368 0 0 nch w=1u l=180n
M4089 nw491 t1553 vdd vdd pch w=2u l=180n
M4090 nw491 t1553 0 0 nch w=1u l=180n
Cnw491 nw491 0 2f
CT1555 t1555 0 0.1f
M4091 t1555 nw296 0 0 nch w=1u l=180n
M4092 t1555 nw371 0 0 nch w=1u l=180n
CT1556 t1556 0 0.1f
M4093 t1556 nw296 vdd vdd pch w=2u l=180n
M4094 t1555 nw371 t1556 vdd pch w=2u l=180n
M4095 nw492 t1555 vdd vdd pch w=2u l=180n
M4096 nw492 t1555 0 0 nch w=1u l=180n
Cnw492 nw492 0 2f
CT1557 t1557 0 0.1f
CT1558 t1558 0 0.1f
CT1559 t1559 0 0.1f
M4097 t1557 nw298 vdd vdd pch w=2u l=180n
M4098 t1557 nw374 vdd vdd pch w=2u l=180n
CT1560 t1560 0 0.1f
M4099 t1557 nw298 t1560 0 nch w=1u l=180n
M4100 t1560 nw374 0 0 nch w=1u l=180n
M4101 t1558 nw298 vdd vdd pch w=2u l=180n
M4102 t1558 t1557 vdd vdd pch w=2u l=180n
CT1561 t1561 0 0.1f
M4103 t1558 nw298 t1561 0 nch w=1u l=180n
M4104 t1561 t1557 0 0 nch w=1u l=180n
M4105 t1559 nw374 vdd vdd pch w=2u l=180n
M4106 t1559 t1557 vdd vdd pch w=2u l=180n
CT1562 t1562 0 0.1f
M4107 t1559 nw374 t1562 0 nch w=1u l=180n
M4108 t1562 t1557 0 0 nch w=1u l=180n
M4109 nw493 t1558 vdd vdd pch w=2u l=180n
M4110 nw493 t1559 vdd vdd pch w=2u l=180n
CT1563 t1563 0 0.1f
M4111 nw493 t1558 t1563 0 nch w=1u l=180n
M4112 t1563 t1559 0 0 nch w=1u l=180n
Cnw493 nw493 0 2f
M4113 nw494 nw300 vdd vdd pch w=2u l=180n
M4114 nw494 nw377 vdd vdd pch w=2u l=180n
CT1564 t1564 0 0.1f
M4115 nw494 nw300 t1564 0 nch w=1u l=180n
M4116 t1564 nw377 0 0 nch w=1u l=180n
Cnw494 nw494 0 2f
M4117 nw495 nw302 0 0 nch w=1u l=180n
M4118 nw495 nw380 0 0 nch w=1u l=180n
CT1565 t1565 0 0.1f
M4119 t1565 nw302 vdd vdd pch w=2u l=180n
M4120 nw495 nw380 t1565 vdd pch w=2u l=180n
Cnw495 nw495 0 2f
CT1566 t1566 0 0.1f
M4121 t1566 nw304 vdd vdd pch w=2u l=180n
M4122 t1566 nw383 vdd vdd pch w=2u l=180n
CT1567 t1567 0 0.1f
M4123 t1566 nw304 t1567 0 nch w=1u l=180n
M4124 t1567 nw383 0 0 nch w=1u l=180n
M4125 nw496 t1566 vdd vdd pch w=2u l=180n
M4126 nw496 t1566 0 0 nch w=1u l=180n
Cnw496 nw496 0 2f
CT1568 t1568 0 0.1f
M4127 t1568 nw306 0 0 nch w=1u l=180n
M4128 t1568 nw386 0 0 nch w=1u l=180n
CT1569 t1569 0 0.1f
M4129 t1569 nw306 vdd vdd pch w=2u l=180n
M4130 t1568 nw386 t1569 vdd pch w=2u l=180n
M4131 nw497 t1568 vdd vdd pch w=2u l=180n
M4132 nw497 t1568 0 0 nch w=1u l=180n
Cnw497 nw497 0 2f
CT1570 t1570 0 0.1f
CT1571 t1571 0 0.1f
CT1572 t1572 0 0.1f
M4133 t1570 nw308 vdd vdd pch w=2u l=180n
M4134 t1570 nw389 vdd vdd pch w=2u l=180n
CT1573 t1573 0 0.1f
M4135 t1570 nw308 t1573 0 nch w=1u l=180n
M4136 t1573 nw389 0 0 nch w=1u l=180n
M4137 t1571 nw308 vdd vdd pch w=2u l=180n
M4138 t1571 t1570 vdd vdd pch w=2u l=180n
CT1574 t1574 0 0.1f
M4139 t1571 nw308 t1574 0 nch w=1u l=180n
M4140 t1574 t1570 0 0 nch w=1u l=180n
M4141 t1572 nw389 vdd vdd pch w=2u l=180n
M4142 t1572 t1570 vdd vdd pch w=2u l=180n
CT1575 t1575 0 0.1f
M4143 t1572 nw389 t1575 0 nch w=1u l=180n
M4144 t1575 t1570 0 0 nch w=1u l=180n
M4145 nw498 t1571 vdd vdd pch w=2u l=180n
M4146 nw498 t1572 vdd vdd pch w=2u l=180n
CT1576 t1576 0 0.1f
M4147 nw498 t1571 t1576 0 nch w=1u l=180n
M4148 t1576 t1572 0 0 nch w=1u l=180n
Cnw498 nw498 0 2f
M4149 nw499 nw310 vdd vdd pch w=2u l=180n
M4150 nw499 nw392 vdd vdd pch w=2u l=180n
CT1577 t1577 0 0.1f
M4151 nw499 nw310 t1577 0 nch w=1u l=180n
M4152 t1577 nw392 0 0 nch w=1u l=180n
Cnw499 nw499 0 2f
M4153 nw500 nw312 0 0 nch w=1u l=180n
M4154 nw500 nw395 0 0 nch w=1u l=180n
CT1578 t1578 0 0.1f
M4155 t1578 nw312 vdd vdd pch w=2u l=180n
M4156 nw500 nw395 t1578 vdd pch w=2u l=180n
Cnw500 nw500 0 2f
CT1579 t1579 0 0.1f
M4157 t1579 nw314 vdd vdd pch w=2u l=180n
M4158 t1579 nw398 vdd vdd pch w=2u l=180n
CT1580 t1580 0 0.1f
M4159 t1579 nw314 t1580 0 nch w=1u l=180n
M4160 t1580 nw398 0 0 nch w=1u l=180n
M4161 nw501 t1579 vdd vdd pch w=2u l=180n
M4162 nw501 t1579 0 0 nch w=1u l=180n
Cnw501 nw501 0 2f
CT1581 t1581 0 0.1f
M4163 t1581 nw316 0 0 nch w=1u l=180n
M4164 t1581 nw401 0 0 nch w=1u l=180n
CT1582 t1582 0 0.1f
M4165 t1582 nw316 vdd vdd pch w=2u l=180n
M4166 t1581 nw401 t1582 vdd pch w=2u l=180n
M4167 nw502 t1581 vdd vdd pch w=2u l=180n
M4168 nw502 t1581 0 0 nch w=1u l=180n
Cnw502 nw502 0 2f
CT1583 t1583 0 0.1f
CT1584 t1584 0 0.1f
CT1585 t1585 0 0.1f
M4169 t1583 nw318 vdd vdd pch w=2u l=180n
M4170 t1583 nw404 vdd vdd pch w=2u l=180n
CT1586 t1586 0 0.1f
M4171 t1583 nw318 t1586 0 nch w=1u l=180n
M4172 t1586 nw404 0 0 nch w=1u l=180n
M4173 t1584 nw318 vdd vdd pch w=2u l=180n
M4174 t1584 t1583 vdd vdd pch w=2u l=180n
CT1587 t1587 0 0.1f
M4175 t1584 nw318 t1587 0 nch w=1u l=180n
M4176 t1587 t1583 0 0 nch w=1u l=180n
M4177 t1585 nw404 vdd vdd pch w=2u l=180n
M4178 t1585 t1583 vdd vdd pch w=2u l=180n
CT1588 t1588 0 0.1f
M4179 t1585 nw404 t1588 0 nch w=1u l=180n
M4180 t1588 t1583 0 0 nch w=1u l=180n
M4181 nw503 t1584 vdd vdd pch w=2u l=180n
M4182 nw503 t1585 vdd vdd pch w=2u l=180n
CT1589 t1589 0 0.1f
M4183 nw503 t1584 t1589 0 nch w=1u l=180n
M4184 t1589 t1585 0 0 nch w=1u l=180n
Cnw503 nw503 0 2f
M4185 nw504 nw320 vdd vdd pch w=2u l=180n
M4186 nw504 nw407 vdd vdd pch w=2u l=180n
CT1590 t1590 0 0.1f
M4187 nw504 nw320 t1590 0 nch w=1u l=180n
M4188 t1590 nw407 0 0 nch w=1u l=180n
Cnw504 nw504 0 2f
M4189 nw505 nw322 0 0 nch w=1u l=180n
M4190 nw505 nw410 0 0 nch w=1u l=180n
CT1591 t1591 0 0.1f
M4191 t1591 nw322 vdd vdd pch w=2u l=180n
M4192 nw505 nw410 t1591 vdd pch w=2u l=180n
Cnw505 nw505 0 2f
CT1592 t1592 0 0.1f
M4193 t1592 nw324 vdd vdd pch w=2u l=180n
M4194 t1592 nw413 vdd vdd pch w=2u l=180n
CT1593 t1593 0 0.1f
M4195 t1592 nw324 t1593 0 nch w=1u l=180n
M4196 t1593 nw413 0 0 nch w=1u l=180n
M4197 nw506 t1592 vdd vdd pch w=2u l=180n
M4198 nw506 t1592 0 0 nch w=1u l=180n
Cnw506 nw506 0 2f
CT1594 t1594 0 0.1f
M4199 t1594 nw326 0 0 nch w=1u l=180n
M4200 t1594 nw416 0 0 nch w=1u l=180n
CT1595 t1595 0 0.1f
M4201 t1595 nw326 vdd vdd pch w=2u l=180n
M4202 t1594 nw416 t1595 vdd pch w=2u l=180n
M4203 nw507 t1594 vdd vdd pch w=2u l=180n
M4204 nw507 t1594 0 0 nch w=1u l=180n
Cnw507 nw507 0 2f
CT1596 t1596 0 0.1f
CT1597 t1597 0 0.1f
CT1598 t1598 0 0.1f
M4205 t1596 nw328 vdd vdd pch w=2u l=180n
M4206 t1596 nw419 vdd vdd pch w=2u l=180n
CT1599 t1599 0 0.1f
M4207 t1596 nw328 t1599 0 nch w=1u l=180n
M4208 t1599 nw419 0 0 nch w=1u l=180n
M4209 t1597 nw328 vdd vdd pch w=2u l=180n
M4210 t1597 t1596 vdd vdd pch w=2u l=180n
CT1600 t1600 0 0.1f
M4211 t1597 nw328 t1600 0 nch w=1u l=180n
M4212 t1600 t1596 0 0 nch w=1u l=180n
M4213 t1598 nw419 vdd vdd pch w=2u l=180n
M4214 t1598 t1596 vdd vdd pch w=2u l=180n
CT1601 t1601 0 0.1f
M4215 t1598 nw419 t1601 0 nch w=1u l=180n
M4216 t1601 t1596 0 0 nch w=1u l=180n
M4217 nw508 t1597 vdd vdd pch w=2u l=180n
M4218 nw508 t1598 vdd vdd pch w=2u l=180n
CT1602 t1602 0 0.1f
M4219 nw508 t1597 t1602 0 nch w=1u l=180n
M4220 t1602 t1598 0 0 nch w=1u l=180n
Cnw508 nw508 0 2f
M4221 nw509 nw330 vdd vdd pch w=2u l=180n
M4222 nw509 nw422 vdd vdd pch w=2u l=180n
CT1603 t1603 0 0.1f
M4223 nw509 nw330 t1603 0 nch w=1u l=180n
M4224 t1603 nw422 0 0 nch w=1u l=180n
Cnw509 nw509 0 2f
M4225 nw510 nw332 0 0 nch w=1u l=180n
M4226 nw510 nw425 0 0 nch w=1u l=180n
CT1604 t1604 0 0.1f
M4227 t1604 nw332 vdd vdd pch w=2u l=180n
M4228 nw510 nw425 t1604 vdd pch w=2u l=180n
Cnw510 nw510 0 2f
CT1605 t1605 0 0.1f
M4229 t1605 nw334 vdd vdd pch w=2u l=180n
M4230 t1605 nw428 vdd vdd pch w=2u l=180n
CT1606 t1606 0 0.1f
M4231 t1605 nw334 t1606 0 nch w=1u l=180n
M4232 t1606 nw428 0 0 nch w=1u l=180n
M4233 nw511 t1605 vdd vdd pch w=2u l=180n
M4234 nw511 t1605 0 0 nch w=1u l=180n
Cnw511 nw511 0 2f
CT1607 t1607 0 0.1f
M4235 t1607 nw336 0 0 nch w=1u l=180n
M4236 t1607 nw431 0 0 nch w=1u l=180n
CT1608 t1608 0 0.1f
M4237 t1608 nw336 vdd vdd pch w=2u l=180n
M4238 t1607 nw431 t1608 vdd pch w=2u l=180n
M4239 nw512 t1607 vdd vdd pch w=2u l=180n
M4240 nw512 t1607 0 0 nch w=1u l=180n
Cnw512 nw512 0 2f
CT1609 t1609 0 0.1f
CT1610 t1610 0 0.1f
CT1611 t1611 0 0.1f
M4241 t1609 nw338 vdd vdd pch w=2u l=180n
M4242 t1609 nw434 vdd vdd pch w=2u l=180n
CT1612 t1612 0 0.1f
M4243 t1609 nw338 t1612 0 nch w=1u l=180n
M4244 t1612 nw434 0 0 nch w=1u l=180n
M4245 t1610 nw338 vdd vdd pch w=2u l=180n
M4246 t1610 t1609 vdd vdd pch w=2u l=180n
CT1613 t1613 0 0.1f
M4247 t1610 nw338 t1613 0 nch w=1u l=180n
M4248 t1613 t1609 0 0 nch w=1u l=180n
M4249 t1611 nw434 vdd vdd pch w=2u l=180n
M4250 t1611 t1609 vdd vdd pch w=2u l=180n
CT1614 t1614 0 0.1f
M4251 t1611 nw434 t1614 0 nch w=1u l=180n
M4252 t1614 t1609 0 0 nch w=1u l=180n
M4253 nw513 t1610 vdd vdd pch w=2u l=180n
M4254 nw513 t1611 vdd vdd pch w=2u l=180n
CT1615 t1615 0 0.1f
M4255 nw513 t1610 t1615 0 nch w=1u l=180n
M4256 t1615 t1611 0 0 nch w=1u l=180n
Cnw513 nw513 0 2f
M4257 nw514 nw340 vdd vdd pch w=2u l=180n
M4258 nw514 nw437 vdd vdd pch w=2u l=180n
CT1616 t1616 0 0.1f
M4259 nw514 nw340 t1616 0 nch w=1u l=180n
M4260 t1616 nw437 0 0 nch w=1u l=180n
Cnw514 nw514 0 2f
M4261 nw515 nw342 0 0 nch w=1u l=180n
M4262 nw515 nw440 0 0 nch w=1u l=180n
CT1617 t1617 0 0.1f
M4263 t1617 nw342 vdd vdd pch w=2u l=180n
M4264 nw515 nw440 t1617 vdd pch w=2u l=180n
Cnw515 nw515 0 2f
CT1618 t1618 0 0.1f
M4265 t1618 nw344 vdd vdd pch w=2u l=180n
M4266 t1618 nw443 vdd vdd pch w=2u l=180n
CT1619 t1619 0 0.1f
M4267 t1618 nw344 t1619 0 nch w=1u l=180n
M4268 t1619 nw443 0 0 nch w=1u l=180n
M4269 nw516 t1618 vdd vdd pch w=2u l=180n
M4270 nw516 t1618 0 0 nch w=1u l=180n
Cnw516 nw516 0 2f
CT1620 t1620 0 0.1f
M4271 t1620 nw346 0 0 nch w=1u l=180n
M4272 t1620 nw446 0 0 nch w=1u l=180n
CT1621 t1621 0 0.1f
M4273 t1621 nw346 vdd vdd pch w=2u l=180n
M4274 t1620 nw446 t1621 vdd pch w=2u l=180n
M4275 nw517 t1620 vdd vdd pch w=2u l=180n
M4276 nw517 t1620 0 0 nch w=1u l=180n
Cnw517 nw517 0 2f
CT1622 t1622 0 0.1f
CT1623 t1623 0 0.1f
CT1624 t1624 0 0.1f
M4277 t1622 nw348 vdd vdd pch w=2u l=180n
M4278 t1622 nw449 vdd vdd pch w=2u l=180n
CT1625 t1625 0 0.1f
M4279 t1622 nw348 t1625 0 nch w=1u l=180n
M4280 t1625 nw449 0 0 nch w=1u l=180n
M4281 t1623 nw348 vdd vdd pch w=2u l=180n
M4282 t1623 t1622 vdd vdd pch w=2u l=180n
CT1626 t1626 0 0.1f
M4283 t1623 nw348 t1626 0 nch w=1u l=180n
M4284 t1626 t1622 0 0 nch w=1u l=180n
M4285 t1624 nw449 vdd vdd pch w=2u l=180n
M4286 t1624 t1622 vdd vdd pch w=2u l=180n
CT1627 t1627 0 0.1f
M4287 t1624 nw449 t1627 0 nch w=1u l=180n
M4288 t1627 t1622 0 0 nch w=1u l=180n
M4289 nw518 t1623 vdd vdd pch w=2u l=180n
M4290 nw518 t1624 vdd vdd pch w=2u l=180n
CT1628 t1628 0 0.1f
M4291 nw518 t1623 t1628 0 nch w=1u l=180n
M4292 t1628 t1624 0 0 nch w=1u l=180n
Cnw518 nw518 0 2f
M4293 nw519 nw350 vdd vdd pch w=2u l=180n
M4294 nw519 nw452 vdd vdd pch w=2u l=180n
CT1629 t1629 0 0.1f
M4295 nw519 nw350 t1629 0 nch w=1u l=180n
M4296 t1629 nw452 0 0 nch w=1u l=180n
Cnw519 nw519 0 2f
M4297 nw520 nw352 0 0 nch w=1u l=180n
M4298 nw520 nw455 0 0 nch w=1u l=180n
CT1630 t1630 0 0.1f
M4299 t1630 nw352 vdd vdd pch w=2u l=180n
M4300 nw520 nw455 t1630 vdd pch w=2u l=180n
Cnw520 nw520 0 2f
CT1631 t1631 0 0.1f
M4301 t1631 nw354 vdd vdd pch w=2u l=180n
M4302 t1631 nw458 vdd vdd pch w=2u l=180n
CT1632 t1632 0 0.1f
M4303 t1631 nw354 t1632 0 nch w=1u l=180n
M4304 t1632 nw458 0 0 nch w=1u l=180n
M4305 nw521 t1631 vdd vdd pch w=2u l=180n
M4306 nw521 t1631 0 0 nch w=1u l=180n
Cnw521 nw521 0 2f
CT1633 t1633 0 0.1f
M4307 t1633 nw356 0 0 nch w=1u l=180n
M4308 t1633 nw461 0 0 nch w=1u l=180n
CT1634 t1634 0 0.1f
M4309 t1634 nw356 vdd vdd pch w=2u l=180n
M4310 t1633 nw461 t1634 vdd pch w=2u l=180n
M4311 nw522 t1633 vdd vdd pch w=2u l=180n
M4312 nw522 t1633 0 0 nch w=1u l=180n
Cnw522 nw522 0 2f
CT1635 t1635 0 0.1f
CT1636 t1636 0 0.1f
CT1637 t1637 0 0.1f
M4313 t1635 nw358 vdd vdd pch w=2u l=180n
M4314 t1635 nw464 vdd vdd pch w=2u l=180n
CT1638 t1638 0 0.1f
M4315 t1635 nw358 t1638 0 nch w=1u l=180n
M4316 t1638 nw464 0 0 nch w=1u l=180n
M4317 t1636 nw358 vdd vdd pch w=2u l=180n
M4318 t1636 t1635 vdd vdd pch w=2u l=180n
CT1639 t1639 0 0.1f
M4319 t1636 nw358 t1639 0 nch w=1u l=180n
M4320 t1639 t1635 0 0 nch w=1u l=180n
M4321 t1637 nw464 vdd vdd pch w=2u l=180n
M4322 t1637 t1635 vdd vdd pch w=2u l=180n
CT1640 t1640 0 0.1f
M4323 t1637 nw464 t1640 0 nch w=1u l=180n
M4324 t1640 t1635 0 0 nch w=1u l=180n
M4325 nw523 t1636 vdd vdd pch w=2u l=180n
M4326 nw523 t1637 vdd vdd pch w=2u l=180n
CT1641 t1641 0 0.1f
M4327 nw523 t1636 t1641 0 nch w=1u l=180n
M4328 t1641 t1637 0 0 nch w=1u l=180n
Cnw523 nw523 0 2f
M4329 nw524 nw360 vdd vdd pch w=2u l=180n
M4330 nw524 nw467 vdd vdd pch w=2u l=180n
CT1642 t1642 0 0.1f
M4331 nw524 nw360 t1642 0 nch w=1u l=180n
M4332 t1642 nw467 0 0 nch w=1u l=180n
Cnw524 nw524 0 2f
M4333 nw525 nw362 0 0 nch w=1u l=180n
M4334 nw525 nw470 0 0 nch w=1u l=180n
CT1643 t1643 0 0.1f
M4335 t1643 nw362 vdd vdd pch w=2u l=180n
M4336 nw525 nw470 t1643 vdd pch w=2u l=180n
Cnw525 nw525 0 2f
CT1644 t1644 0 0.1f
M4337 t1644 nw364 vdd vdd pch w=2u l=180n
M4338 t1644 nw473 vdd vdd pch w=2u l=180n
CT1645 t1645 0 0.1f
M4339 t1644 nw364 t1645 0 nch w=1u l=180n
M4340 t1645 nw473 0 0 nch w=1u l=180n
M4341 nw526 t1644 vdd vdd pch w=2u l=180n
M4342 nw526 t1644 0 0 nch w=1u l=180n
Cnw526 nw526 0 2f
CT1646 t1646 0 0.1f
M4343 t1646 nw366 0 0 nch w=1u l=180n
M4344 t1646 nw476 0 0 nch w=1u l=180n
CT1647 t1647 0 0.1f
M4345 t1647 nw366 vdd vdd pch w=2u l=180n
M4346 t1646 nw476 t1647 vdd pch w=2u l=180n
M4347 nw527 t1646 vdd vdd pch w=2u l=180n
M4348 nw527 t1646 0 0 nch w=1u l=180n
Cnw527 nw527 0 2f
CT1648 t1648 0 0.1f
CT1649 t1649 0 0.1f
CT1650 t1650 0 0.1f
M4349 t1648 nw368 vdd vdd pch w=2u l=180n
M4350 t1648 nw479 vdd vdd pch w=2u l=180n
CT1651 t1651 0 0.1f
M4351 t1648 nw368 t1651 0 nch w=1u l=180n
M4352 t1651 nw479 0 0 nch w=1u l=180n
M4353 t1649 nw368 vdd vdd pch w=2u l=180n
M4354 t1649 t1648 vdd vdd pch w=2u l=180n
CT1652 t1652 0 0.1f
M4355 t1649 nw368 t1652 0 nch w=1u l=180n
M4356 t1652 t1648 0 0 nch w=1u l=180n
M4357 t1650 nw479 vdd vdd pch w=2u l=180n
M4358 t1650 t1648 vdd vdd pch w=2u l=180n
CT1653 t1653 0 0.1f
M4359 t1650 nw479 t1653 0 nch w=1u l=180n
M4360 t1653 t1648 0 0 nch w=1u l=180n
M4361 nw528 t1649 vdd vdd pch w=2u l=180n
M4362 nw528 t1650 vdd vdd pch w=2u l=180n
CT1654 t1654 0 0.1f
M4363 nw528 t1649 t1654 0 nch w=1u l=180n
M4364 t1654 t1650 0 0 nch w=1u l=180n
Cnw528 nw528 0 2f
M4365 nw529 nw370 vdd vdd pch w=2u l=180n
M4366 nw529 nw482 vdd vdd pch w=2u l=180n
CT1655 t1655 0 0.1f
M4367 nw529 nw370 t1655 0 nch w=1u l=180n
M4368 t1655 nw482 0 0 nch w=1u l=180n
Cnw529 nw529 0 2f
M4369 nw530 nw372 0 0 nch w=1u l=180n
M4370 nw530 nw485 0 0 nch w=1u l=180n
CT1656 t1656 0 0.1f
M4371 t1656 nw372 vdd vdd pch w=2u l=180n
M4372 nw530 nw485 t1656 vdd pch w=2u l=180n
Cnw530 nw530 0 2f
CT1657 t1657 0 0.1f
M4373 t1657 nw374 vdd vdd pch w=2u l=180n
M4374 t1657 nw488 vdd vdd pch w=2u l=180n
CT1658 t1658 0 0.1f
M4375 t1657 nw374 t1658 0 nch w=1u l=180n
M4376 t1658 nw488 0 0 nch w=1u l=180n
M4377 nw531 t1657 vdd vdd pch w=2u l=180n
M4378 nw531 t1657 0 0 nch w=1u l=180n
Cnw531 nw531 0 2f
CT1659 t1659 0 0.1f
M4379 t1659 nw376 0 0 nch w=1u l=180n
M4380 t1659 nw491 0 0 nch w=1u l=180n
CT1660 t1660 0 0.1f
M4381 t1660 nw376 vdd vdd pch w=2u l=180n
M4382 t1659 nw491 t1660 vdd pch w=2u l=180n
M4383 nw532 t1659 vdd vdd pch w=2u l=180n
M4384 nw532 t1659 0 0 nch w=1u l=180n
Cnw532 nw532 0 2f
CT1661 t1661 0 0.1f
CT1662 t1662 0 0.1f
CT1663 t1663 0 0.1f
M4385 t1661 nw378 vdd vdd pch w=2u l=180n
M4386 t1661 nw494 vdd vdd pch w=2u l=180n
CT1664 t1664 0 0.1f
M4387 t1661 nw378 t1664 0 nch w=1u l=180n
M4388 t1664 nw494 0 0 nch w=1u l=180n
M4389 t1662 nw378 vdd vdd pch w=2u l=180n
M4390 t1662 t1661 vdd vdd pch w=2u l=180n
CT1665 t1665 0 0.1f
M4391 t1662 nw378 t1665 0 nch w=1u l=180n
M4392 t1665 t1661 0 0 nch w=1u l=180n
M4393 t1663 nw494 vdd vdd pch w=2u l=180n
M4394 t1663 t1661 vdd vdd pch w=2u l=180n
CT1666 t1666 0 0.1f
M4395 t1663 nw494 t1666 0 nch w=1u l=180n
M4396 t1666 t1661 0 0 nch w=1u l=180n
M4397 nw533 t1662 vdd vdd pch w=2u l=180n
M4398 nw533 t1663 vdd vdd pch w=2u l=180n
CT1667 t1667 0 0.1f
M4399 nw533 t1662 t1667 0 nch w=1u l=180n
M4400 t1667 t1663 0 0 nch w=1u l=180n
Cnw533 nw533 0 2f
M4401 nw534 nw380 vdd vdd pch w=2u l=180n
M4402 nw534 nw497 vdd vdd pch w=2u l=180n
CT1668 t1668 0 0.1f
M4403 nw534 nw380 t1668 0 nch w=1u l=180n
M4404 t1668 nw497 0 0 nch w=1u l=180n
Cnw534 nw534 0 2f
M4405 nw535 nw382 0 0 nch w=1u l=180n
M4406 nw535 nw500 0 0 nch w=1u l=180n
CT1669 t1669 0 0.1f
M4407 t1669 nw382 vdd vdd pch w=2u l=180n
M4408 nw535 nw500 t1669 vdd pch w=2u l=180n
Cnw535 nw535 0 2f
CT1670 t1670 0 0.1f
M4409 t1670 nw384 vdd vdd pch w=2u l=180n
M4410 t1670 nw503 vdd vdd pch w=2u l=180n
CT1671 t1671 0 0.1f
M4411 t1670 nw384 t1671 0 nch w=1u l=180n
M4412 t1671 nw503 0 0 nch w=1u l=180n
M4413 nw536 t1670 vdd vdd pch w=2u l=180n
M4414 nw536 t1670 0 0 nch w=1u l=180n
Cnw536 nw536 0 2f
CT1672 t1672 0 0.1f
M4415 t1672 nw386 0 0 nch w=1u l=180n
M4416 t1672 nw506 0 0 nch w=1u l=180n
CT1673 t1673 0 0.1f
M4417 t1673 nw386 vdd vdd pch w=2u l=180n
M4418 t1672 nw506 t1673 vdd pch w=2u l=180n
M4419 nw537 t1672 vdd vdd pch w=2u l=180n
M4420 nw537 t1672 0 0 nch w=1u l=180n
Cnw537 nw537 0 2f
CT1674 t1674 0 0.1f
CT1675 t1675 0 0.1f
CT1676 t1676 0 0.1f
M4421 t1674 nw388 vdd vdd pch w=2u l=180n
M4422 t1674 nw509 vdd vdd pch w=2u l=180n
CT1677 t1677 0 0.1f
M4423 t1674 nw388 t1677 0 nch w=1u l=180n
M4424 t1677 nw509 0 0 nch w=1u l=180n
M4425 t1675 nw388 vdd vdd pch w=2u l=180n
M4426 t1675 t1674 vdd vdd pch w=2u l=180n
CT1678 t1678 0 0.1f
M4427 t1675 nw388 t1678 0 nch w=1u l=180n
M4428 t1678 t1674 0 0 nch w=1u l=180n
M4429 t1676 nw509 vdd vdd pch w=2u l=180n
M4430 t1676 t1674 vdd vdd pch w=2u l=180n
CT1679 t1679 0 0.1f
M4431 t1676 nw509 t1679 0 nch w=1u l=180n
M4432 t1679 t1674 0 0 nch w=1u l=180n
M4433 nw538 t1675 vdd vdd pch w=2u l=180n
M4434 nw538 t1676 vdd vdd pch w=2u l=180n
CT1680 t1680 0 0.1f
M4435 nw538 t1675 t1680 0 nch w=1u l=180n
M4436 t1680 t1676 0 0 nch w=1u l=180n
Cnw538 nw538 0 2f
M4437 nw539 nw390 vdd vdd pch w=2u l=180n
M4438 nw539 nw512 vdd vdd pch w=2u l=180n
CT1681 t1681 0 0.1f
M4439 nw539 nw390 t1681 0 nch w=1u l=180n
M4440 t1681 nw512 0 0 nch w=1u l=180n
Cnw539 nw539 0 2f
M4441 nw540 nw392 0 0 nch w=1u l=180n
M4442 nw540 nw515 0 0 nch w=1u l=180n
CT1682 t1682 0 0.1f
M4443 t1682 nw392 vdd vdd pch w=2u l=180n
M4444 nw540 nw515 t1682 vdd pch w=2u l=180n
Cnw540 nw540 0 2f
CT1683 t1683 0 0.1f
M4445 t1683 nw394 vdd vdd pch w=2u l=180n
M4446 t1683 nw518 vdd vdd pch w=2u l=180n
CT1684 t1684 0 0.1f
M4447 t1683 nw394 t1684 0 nch w=1u l=180n
M4448 t1684 nw518 0 0 nch w=1u l=180n
M4449 nw541 t1683 vdd vdd pch w=2u l=180n
M4450 nw541 t1683 0 0 nch w=1u l=180n
Cnw541 nw541 0 2f
CT1685 t1685 0 0.1f
M4451 t1685 nw396 0 0 nch w=1u l=180n
M4452 t1685 nw521 0 0 nch w=1u l=180n
CT1686 t1686 0 0.1f
M4453 t1686 nw396 vdd vdd pch w=2u l=180n
M4454 t1685 nw521 t1686 vdd pch w=2u l=180n
M4455 nw542 t1685 vdd vdd pch w=2u l=180n
M4456 nw542 t1685 0 0 nch w=1u l=180n
Cnw542 nw542 0 2f
CT1687 t1687 0 0.1f
CT1688 t1688 0 0.1f
CT1689 t1689 0 0.1f
M4457 t1687 nw398 vdd vdd pch w=2u l=180n
M4458 t1687 nw524 vdd vdd pch w=2u l=180n
CT1690 t1690 0 0.1f
M4459 t1687 nw398 t1690 0 nch w=1u l=180n
M4460 t1690 nw524 0 0 nch w=1u l=180n
M4461 t1688 nw398 vdd vdd pch w=2u l=180n
M4462 t1688 t1687 vdd vdd pch w=2u l=180n
CT1691 t1691 0 0.1f
M4463 t1688 nw398 t1691 0 nch w=1u l=180n
M4464 t1691 t1687 0 0 nch w=1u l=180n
M4465 t1689 nw524 vdd vdd pch w=2u l=180n
M4466 t1689 t1687 vdd vdd pch w=2u l=180n
CT1692 t1692 0 0.1f
M4467 t1689 nw524 t1692 0 nch w=1u l=180n
M4468 t1692 t1687 0 0 nch w=1u l=180n
M4469 nw543 t1688 vdd vdd pch w=2u l=180n
M4470 nw543 t1689 vdd vdd pch w=2u l=180n
CT1693 t1693 0 0.1f
M4471 nw543 t1688 t1693 0 nch w=1u l=180n
M4472 t1693 t1689 0 0 nch w=1u l=180n
Cnw543 nw543 0 2f
M4473 nw544 nw400 vdd vdd pch w=2u l=180n
M4474 nw544 nw527 vdd vdd pch w=2u l=180n
CT1694 t1694 0 0.1f
M4475 nw544 nw400 t1694 0 nch w=1u l=180n
M4476 t1694 nw527 0 0 nch w=1u l=180n
Cnw544 nw544 0 2f
M4477 nw545 nw402 0 0 nch w=1u l=180n
M4478 nw545 nw530 0 0 nch w=1u l=180n
CT1695 t1695 0 0.1f
M4479 t1695 nw402 vdd vdd pch w=2u l=180n
M4480 nw545 nw530 t1695 vdd pch w=2u l=180n
Cnw545 nw545 0 2f
CT1696 t1696 0 0.1f
M4481 t1696 nw404 vdd vdd pch w=2u l=180n
M4482 t1696 nw533 vdd vdd pch w=2u l=180n
CT1697 t1697 0 0.1f
M4483 t1696 nw404 t1697 0 nch w=1u l=180n
M4484 t1697 nw533 0 0 nch w=1u l=180n
M4485 nw546 t1696 vdd vdd pch w=2u l=180n
M4486 nw546 t1696 0 0 nch w=1u l=180n
Cnw546 nw546 0 2f
CT1698 t1698 0 0.1f
M4487 t1698 nw406 0 0 nch w=1u l=180n
M4488 t1698 nw536 0 0 nch w=1u l=180n
CT1699 t1699 0 0.1f
M4489 t1699 nw406 vdd vdd pch w=2u l=180n
M4490 t1698 nw536 t1699 vdd pch w=2u l=180n
M4491 nw547 t1698 vdd vdd pch w=2u l=180n
M4492 nw547 t1698 0 0 nch w=1u l=180n
Cnw547 nw547 0 2f
CT1700 t1700 0 0.1f
CT1701 t1701 0 0.1f
CT1702 t1702 0 0.1f
M4493 t1700 nw408 vdd vdd pch w=2u l=180n
M4494 t1700 nw539 vdd vdd pch w=2u l=180n
CT1703 t1703 0 0.1f
M4495 t1700 nw408 t1703 0 nch w=1u l=180n
M4496 t1703 nw539 0 0 nch w=1u l=180n
M4497 t1701 nw408 vdd vdd pch w=2u l=180n
M4498 t1701 t1700 vdd vdd pch w=2u l=180n
CT1704 t1704 0 0.1f
M4499 t1701 nw408 t1704 0 nch w=1u l=180n
M4500 t1704 t1700 0 0 nch w=1u l=180n
M4501 t1702 nw539 vdd vdd pch w=2u l=180n
M4502 t1702 t1700 vdd vdd pch w=2u l=180n
CT1705 t1705 0 0.1f
M4503 t1702 nw539 t1705 0 nch w=1u l=180n
M4504 t1705 t1700 0 0 nch w=1u l=180n
M4505 nw548 t1701 vdd vdd pch w=2u l=180n
M4506 nw548 t1702 vdd vdd pch w=2u l=180n
CT1706 t1706 0 0.1f
M4507 nw548 t1701 t1706 0 nch w=1u l=180n
M4508 t1706 t1702 0 0 nch w=1u l=180n
Cnw548 nw548 0 2f
M4509 nw549 nw410 vdd vdd pch w=2u l=180n
M4510 nw549 nw542 vdd vdd pch w=2u l=180n
CT1707 t1707 0 0.1f
M4511 nw549 nw410 t1707 0 nch w=1u l=180n
M4512 t1707 nw542 0 0 nch w=1u l=180n
Cnw549 nw549 0 2f
M4513 nw550 nw412 0 0 nch w=1u l=180n
M4514 nw550 nw545 0 0 nch w=1u l=180n
CT1708 t1708 0 0.1f
M4515 t1708 nw412 vdd vdd pch w=2u l=180n
M4516 nw550 nw545 t1708 vdd pch w=2u l=180n
Cnw550 nw550 0 2f
CT1709 t1709 0 0.1f
M4517 t1709 nw414 vdd vdd pch w=2u l=180n
M4518 t1709 nw548 vdd vdd pch w=2u l=180n
CT1710 t1710 0 0.1f
M4519 t1709 nw414 t1710 0 nch w=1u l=180n
M4520 t1710 nw548 0 0 nch w=1u l=180n
M4521 nw551 t1709 vdd vdd pch w=2u l=180n
M4522 nw551 t1709 0 0 nch w=1u l=180n
Cnw551 nw551 0 2f
CT1711 t1711 0 0.1f
M4523 t1711 nw416 0 0 nch w=1u l=180n
M4524 t1711 nw551 0 0 nch w=1u l=180n
CT1712 t1712 0 0.1f
M4525 t1712 nw416 vdd vdd pch w=2u l=180n
M4526 t1711 nw551 t1712 vdd pch w=2u l=180n
M4527 nw552 t1711 vdd vdd pch w=2u l=180n
M4528 nw552 t1711 0 0 nch w=1u l=180n
Cnw552 nw552 0 2f
CT1713 t1713 0 0.1f
CT1714 t1714 0 0.1f
CT1715 t1715 0 0.1f
M4529 t1713 nw418 vdd vdd pch w=2u l=180n
M4530 t1713 nq1 vdd vdd pch w=2u l=180n
CT1716 t1716 0 0.1f
M4531 t1713 nw418 t1716 0 nch w=1u l=180n
M4532 t1716 nq1 0 0 nch w=1u l=180n
M4533 t1714 nw418 vdd vdd pch w=2u l=180n
M4534 t1714 t1713 vdd vdd pch w=2u l=180n
CT1717 t1717 0 0.1f
M4535 t1714 nw418 t1717 0 nch w=1u l=180n
M4536 t1717 t1713 0 0 nch w=1u l=180n
M4537 t1715 nq1 vdd vdd pch w=2u l=180n
M4538 t1715 t1713 vdd vdd pch w=2u l=180n
CT1718 t1718 0 0.1f
M4539 t1715 nq1 t1718 0 nch w=1u l=180n
M4540 t1718 t1713 0 0 nch w=1u l=180n
M4541 nw553 t1714 vdd vdd pch w=2u l=180n
M4542 nw553 t1715 vdd vdd pch w=2u l=180n
CT1719 t1719 0 0.1f
M4543 nw553 t1714 t1719 0 nch w=1u l=180n
M4544 t1719 t1715 0 0 nch w=1u l=180n
Cnw553 nw553 0 2f
M4545 nw554 nw420 vdd vdd pch w=2u l=180n
M4546 nw554 nq3 vdd vdd pch w=2u l=180n
CT1720 t1720 0 0.1f
M4547 nw554 nw420 t1720 0 nch w=1u l=180n
M4548 t1720 nq3 0 0 nch w=1u l=180n
Cnw554 nw554 0 2f
M4549 nw555 nw422 0 0 nch w=1u l=180n
M4550 nw555 nq5 0 0 nch w=1u l=180n
CT1721 t1721 0 0.1f
M4551 t1721 nw422 vdd vdd pch w=2u l=180n
M4552 nw555 nq5 t1721 vdd pch w=2u l=180n
Cnw555 nw555 0 2f
CT1722 t1722 0 0.1f
M4553 t1722 nw424 vdd vdd pch w=2u l=180n
M4554 t1722 nq7 vdd vdd pch w=2u l=180n
CT1723 t1723 0 0.1f
M4555 t1722 nw424 t1723 0 nch w=1u l=180n
M4556 t1723 nq7 0 0 nch w=1u l=180n
M4557 nw556 t1722 vdd vdd pch w=2u l=180n
M4558 nw556 t1722 0 0 nch w=1u l=180n
Cnw556 nw556 0 2f
CT1724 t1724 0 0.1f
M4559 t1724 nw426 0 0 nch w=1u l=180n
M4560 t1724 nq9 0 0 nch w=1u l=180n
CT1725 t1725 0 0.1f
M4561 t1725 nw426 vdd vdd pch w=2u l=180n
M4562 t1724 nq9 t1725 vdd pch w=2u l=180n
M4563 nw557 t1724 vdd vdd pch w=2u l=180n
M4564 nw557 t1724 0 0 nch w=1u l=180n
Cnw557 nw557 0 2f
CT1726 t1726 0 0.1f
CT1727 t1727 0 0.1f
CT1728 t1728 0 0.1f
M4565 t1726 nw428 vdd vdd pch w=2u l=180n
M4566 t1726 nq11 vdd vdd pch w=2u l=180n
CT1729 t1729 0 0.1f
M4567 t1726 nw428 t1729 0 nch w=1u l=180n
M4568 t1729 nq11 0 0 nch w=1u l=180n
M4569 t1727 nw428 vdd vdd pch w=2u l=180n
M4570 t1727 t1726 vdd vdd pch w=2u l=180n
CT1730 t1730 0 0.1f
M4571 t1727 nw428 t1730 0 nch w=1u l=180n
M4572 t1730 t1726 0 0 nch w=1u l=180n
M4573 t1728 nq11 vdd vdd pch w=2u l=180n
M4574 t1728 t1726 vdd vdd pch w=2u l=180n
CT1731 t1731 0 0.1f
M4575 t1728 nq11 t1731 0 nch w=1u l=180n
M4576 t1731 t1726 0 0 nch w=1u l=180n
M4577 nw558 t1727 vdd vdd pch w=2u l=180n
M4578 nw558 t1728 vdd vdd pch w=2u l=180n
CT1732 t1732 0 0.1f
M4579 nw558 t1727 t1732 0 nch w=1u l=180n
M4580 t1732 t1728 0 0 nch w=1u l=180n
Cnw558 nw558 0 2f
M4581 nw559 nw430 vdd vdd pch w=2u l=180n
M4582 nw559 nq13 vdd vdd pch w=2u l=180n
CT1733 t1733 0 0.1f
M4583 nw559 nw430 t1733 0 nch w=1u l=180n
M4584 t1733 nq13 0 0 nch w=1u l=180n
Cnw559 nw559 0 2f
M4585 nw560 nw432 0 0 nch w=1u l=180n
M4586 nw560 nq15 0 0 nch w=1u l=180n
CT1734 t1734 0 0.1f
M4587 t1734 nw432 vdd vdd pch w=2u l=180n
M4588 nw560 nq15 t1734 vdd pch w=2u l=180n
Cnw560 nw560 0 2f
CT1735 t1735 0 0.1f
M4589 t1735 nw434 vdd vdd pch w=2u l=180n
M4590 t1735 nq17 vdd vdd pch w=2u l=180n
CT1736 t1736 0 0.1f
M4591 t1735 nw434 t1736 0 nch w=1u l=180n
M4592 t1736 nq17 0 0 nch w=1u l=180n
M4593 nw561 t1735 vdd vdd pch w=2u l=180n
M4594 nw561 t1735 0 0 nch w=1u l=180n
Cnw561 nw561 0 2f
CT1737 t1737 0 0.1f
M4595 t1737 nw436 0 0 nch w=1u l=180n
M4596 t1737 nq19 0 0 nch w=1u l=180n
CT1738 t1738 0 0.1f
M4597 t1738 nw436 vdd vdd pch w=2u l=180n
M4598 t1737 nq19 t1738 vdd pch w=2u l=180n
M4599 nw562 t1737 vdd vdd pch w=2u l=180n
M4600 nw562 t1737 0 0 nch w=1u l=180n
Cnw562 nw562 0 2f
CT1739 t1739 0 0.1f
CT1740 t1740 0 0.1f
CT1741 t1741 0 0.1f
M4601 t1739 nw438 vdd vdd pch w=2u l=180n
M4602 t1739 nq21 vdd vdd pch w=2u l=180n
CT1742 t1742 0 0.1f
M4603 t1739 nw438 t1742 0 nch w=1u l=180n
M4604 t1742 nq21 0 0 nch w=1u l=180n
M4605 t1740 nw438 vdd vdd pch w=2u l=180n
M4606 t1740 t1739 vdd vdd pch w=2u l=180n
CT1743 t1743 0 0.1f
M4607 t1740 nw438 t1743 0 nch w=1u l=180n
M4608 t1743 t1739 0 0 nch w=1u l=180n
M4609 t1741 nq21 vdd vdd pch w=2u l=180n
M4610 t1741 t1739 vdd vdd pch w=2u l=180n
CT1744 t1744 0 0.1f
M4611 t1741 nq21 t1744 0 nch w=1u l=180n
M4612 t1744 t1739 0 0 nch w=1u l=180n
M4613 nw563 t1740 vdd vdd pch w=2u l=180n
M4614 nw563 t1741 vdd vdd pch w=2u l=180n
CT1745 t1745 0 0.1f
M4615 nw563 t1740 t1745 0 nch w=1u l=180n
M4616 t1745 t1741 0 0 nch w=1u l=180n
Cnw563 nw563 0 2f
M4617 nw564 nw440 vdd vdd pch w=2u l=180n
M4618 nw564 nq23 vdd vdd pch w=2u l=180n
CT1746 t1746 0 0.1f
M4619 nw564 nw440 t1746 0 nch w=1u l=180n
M4620 t1746 nq23 0 0 nch w=1u l=180n
Cnw564 nw564 0 2f
M4621 nw565 nw442 0 0 nch w=1u l=180n
M4622 nw565 nq25 0 0 nch w=1u l=180n
CT1747 t1747 0 0.1f
M4623 t1747 nw442 vdd vdd pch w=2u l=180n
M4624 nw565 nq25 t1747 vdd pch w=2u l=180n
Cnw565 nw565 0 2f
CT1748 t1748 0 0.1f
M4625 t1748 nw444 vdd vdd pch w=2u l=180n
M4626 t1748 nq27 vdd vdd pch w=2u l=180n
CT1749 t1749 0 0.1f
M4627 t1748 nw444 t1749 0 nch w=1u l=180n
M4628 t1749 nq27 0 0 nch w=1u l=180n
M4629 nw566 t1748 vdd vdd pch w=2u l=180n
M4630 nw566 t1748 0 0 nch w=1u l=180n
Cnw566 nw566 0 2f
CT1750 t1750 0 0.1f
M4631 t1750 nw446 0 0 nch w=1u l=180n
M4632 t1750 nq29 0 0 nch w=1u l=180n
CT1751 t1751 0 0.1f
M4633 t1751 nw446 vdd vdd pch w=2u l=180n
M4634 t1750 nq29 t1751 vdd pch w=2u l=180n
M4635 nw567 t1750 vdd vdd pch w=2u l=180n
M4636 nw567 t1750 0 0 nch w=1u l=180n
Cnw567 nw567 0 2f
CT1752 t1752 0 0.1f
CT1753 t1753 0 0.1f
CT1754 t1754 0 0.1f
M4637 t1752 nw448 vdd vdd pch w=2u l=180n
M4638 t1752 nq31 vdd vdd pch w=2u l=180n
CT1755 t1755 0 0.1f
M4639 t1752 nw448 t1755 0 nch w=1u l=180n
M4640 t1755 nq31 0 0 nch w=1u l=180n
M4641 t1753 nw448 vdd vdd pch w=2u l=180n
M4642 t1753 t1752 vdd vdd pch w=2u l=180n
CT1756 t1756 0 0.1f
M4643 t1753 nw448 t1756 0 nch w=1u l=180n
M4644 t1756 t1752 0 0 nch w=1u l=180n
M4645 t1754 nq31 vdd vdd pch w=2u l=180n
M4646 t1754 t1752 vdd vdd pch w=2u l=180n
CT1757 t1757 0 0.1f
M4647 t1754 nq31 t1757 0 nch w=1u l=180n
M4648 t1757 t1752 0 0 nch w=1u l=180n
M4649 nw568 t1753 vdd vdd pch w=2u l=180n
M4650 nw568 t1754 vdd vdd pch w=2u l=180n
CT1758 t1758 0 0.1f
M4651 nw568 t1753 t1758 0 nch w=1u l=180n
M4652 t1758 t1754 0 0 nch w=1u l=180n
Cnw568 nw568 0 2f
M4653 nw569 nw450 vdd vdd pch w=2u l=180n
M4654 nw569 nq33 vdd vdd pch w=2u l=180n
CT1759 t1759 0 0.1f
M4655 nw569 nw450 t1759 0 nch w=1u l=180n
M4656 t1759 nq33 0 0 nch w=1u l=180n
Cnw569 nw569 0 2f
M4657 nw570 nw452 0 0 nch w=1u l=180n
M4658 nw570 nq35 0 0 nch w=1u l=180n
CT1760 t1760 0 0.1f
M4659 t1760 nw452 vdd vdd pch w=2u l=180n
M4660 nw570 nq35 t1760 vdd pch w=2u l=180n
Cnw570 nw570 0 2f
CT1761 t1761 0 0.1f
M4661 t1761 nw454 vdd vdd pch w=2u l=180n
M4662 t1761 nq37 vdd vdd pch w=2u l=180n
CT1762 t1762 0 0.1f
M4663 t1761 nw454 t1762 0 nch w=1u l=180n
M4664 t1762 nq37 0 0 nch w=1u l=180n
M4665 nw571 t1761 vdd vdd pch w=2u l=180n
M4666 nw571 t1761 0 0 nch w=1u l=180n
Cnw571 nw571 0 2f
CT1763 t1763 0 0.1f
M4667 t1763 nw456 0 0 nch w=1u l=180n
M4668 t1763 nq39 0 0 nch w=1u l=180n
CT1764 t1764 0 0.1f
M4669 t1764 nw456 vdd vdd pch w=2u l=180n
M4670 t1763 nq39 t1764 vdd pch w=2u l=180n
M4671 nw572 t1763 vdd vdd pch w=2u l=180n
M4672 nw572 t1763 0 0 nch w=1u l=180n
Cnw572 nw572 0 2f
CT1765 t1765 0 0.1f
CT1766 t1766 0 0.1f
CT1767 t1767 0 0.1f
M4673 t1765 nw458 vdd vdd pch w=2u l=180n
M4674 t1765 nq41 vdd vdd pch w=2u l=180n
CT1768 t1768 0 0.1f
M4675 t1765 nw458 t1768 0 nch w=1u l=180n
M4676 t1768 nq41 0 0 nch w=1u l=180n
M4677 t1766 nw458 vdd vdd pch w=2u l=180n
M4678 t1766 t1765 vdd vdd pch w=2u l=180n
CT1769 t1769 0 0.1f
M4679 t1766 nw458 t1769 0 nch w=1u l=180n
M4680 t1769 t1765 0 0 nch w=1u l=180n
M4681 t1767 nq41 vdd vdd pch w=2u l=180n
M4682 t1767 t1765 vdd vdd pch w=2u l=180n
CT1770 t1770 0 0.1f
M4683 t1767 nq41 t1770 0 nch w=1u l=180n
M4684 t1770 t1765 0 0 nch w=1u l=180n
M4685 nw573 t1766 vdd vdd pch w=2u l=180n
M4686 nw573 t1767 vdd vdd pch w=2u l=180n
CT1771 t1771 0 0.1f
M4687 nw573 t1766 t1771 0 nch w=1u l=180n
M4688 t1771 t1767 0 0 nch w=1u l=180n
Cnw573 nw573 0 2f
M4689 nw574 nw460 vdd vdd pch w=2u l=180n
M4690 nw574 nq43 vdd vdd pch w=2u l=180n
CT1772 t1772 0 0.1f
M4691 nw574 nw460 t1772 0 nch w=1u l=180n
M4692 t1772 nq43 0 0 nch w=1u l=180n
Cnw574 nw574 0 2f
M4693 nw575 nw462 0 0 nch w=1u l=180n
M4694 nw575 nq45 0 0 nch w=1u l=180n
CT1773 t1773 0 0.1f
M4695 t1773 nw462 vdd vdd pch w=2u l=180n
M4696 nw575 nq45 t1773 vdd pch w=2u l=180n
Cnw575 nw575 0 2f
CT1774 t1774 0 0.1f
M4697 t1774 nw464 vdd vdd pch w=2u l=180n
M4698 t1774 nq47 vdd vdd pch w=2u l=180n
CT1775 t1775 0 0.1f
M4699 t1774 nw464 t1775 0 nch w=1u l=180n
M4700 t1775 nq47 0 0 nch w=1u l=180n
M4701 nw576 t1774 vdd vdd pch w=2u l=180n
M4702 nw576 t1774 0 0 nch w=1u l=180n
Cnw576 nw576 0 2f
CT1776 t1776 0 0.1f
M4703 t1776 nw466 0 0 nch w=1u l=180n
M4704 t1776 nq49 0 0 nch w=1u l=180n
CT1777 t1777 0 0.1f
M4705 t1777 nw466 vdd vdd pch w=2u l=180n
M4706 t1776 nq49 t1777 vdd pch w=2u l=180n
M4707 nw577 t1776 vdd vdd pch w=2u l=180n
M4708 nw577 t1776 0 0 nch w=1u l=180n
Cnw577 nw577 0 2f
CT1778 t1778 0 0.1f
CT1779 t1779 0 0.1f
CT1780 t1780 0 0.1f
M4709 t1778 nw468 vdd vdd pch w=2u l=180n
M4710 t1778 nq51 vdd vdd pch w=2u l=180n
CT1781 t1781 0 0.1f
M4711 t1778 nw468 t1781 0 nch w=1u l=180n
M4712 t1781 nq51 0 0 nch w=1u l=180n
M4713 t1779 nw468 vdd vdd pch w=2u l=180n
M4714 t1779 t1778 vdd vdd pch w=2u l=180n
CT1782 t1782 0 0.1f
M4715 t1779 nw468 t1782 0 nch w=1u l=180n
M4716 t1782 t1778 0 0 nch w=1u l=180n
M4717 t1780 nq51 vdd vdd pch w=2u l=180n
M4718 t1780 t1778 vdd vdd pch w=2u l=180n
CT1783 t1783 0 0.1f
M4719 t1780 nq51 t1783 0 nch w=1u l=180n
M4720 t1783 t1778 0 0 nch w=1u l=180n
M4721 nw578 t1779 vdd vdd pch w=2u l=180n
M4722 nw578 t1780 vdd vdd pch w=2u l=180n
CT1784 t1784 0 0.1f
M4723 nw578 t1779 t1784 0 nch w=1u l=180n
M4724 t1784 t1780 0 0 nch w=1u l=180n
Cnw578 nw578 0 2f
M4725 nw579 nw470 vdd vdd pch w=2u l=180n
M4726 nw579 nq53 vdd vdd pch w=2u l=180n
CT1785 t1785 0 0.1f
M4727 nw579 nw470 t1785 0 nch w=1u l=180n
M4728 t1785 nq53 0 0 nch w=1u l=180n
Cnw579 nw579 0 2f
M4729 nw580 nw472 0 0 nch w=1u l=180n
M4730 nw580 nq55 0 0 nch w=1u l=180n
CT1786 t1786 0 0.1f
M4731 t1786 nw472 vdd vdd pch w=2u l=180n
M4732 nw580 nq55 t1786 vdd pch w=2u l=180n
Cnw580 nw580 0 2f
CT1787 t1787 0 0.1f
M4733 t1787 nw474 vdd vdd pch w=2u l=180n
M4734 t1787 nq57 vdd vdd pch w=2u l=180n
CT1788 t1788 0 0.1f
M4735 t1787 nw474 t1788 0 nch w=1u l=180n
M4736 t1788 nq57 0 0 nch w=1u l=180n
M4737 nw581 t1787 vdd vdd pch w=2u l=180n
M4738 nw581 t1787 0 0 nch w=1u l=180n
Cnw581 nw581 0 2f
CT1789 t1789 0 0.1f
M4739 t1789 nw476 0 0 nch w=1u l=180n
M4740 t1789 nq59 0 0 nch w=1u l=180n
CT1790 t1790 0 0.1f
M4741 t1790 nw476 vdd vdd pch w=2u l=180n
M4742 t1789 nq59 t1790 vdd pch w=2u l=180n
M4743 nw582 t1789 vdd vdd pch w=2u l=180n
M4744 nw582 t1789 0 0 nch w=1u l=180n
Cnw582 nw582 0 2f
CT1791 t1791 0 0.1f
CT1792 t1792 0 0.1f
CT1793 t1793 0 0.1f
M4745 t1791 nw478 vdd vdd pch w=2u l=180n
M4746 t1791 nq61 vdd vdd pch w=2u l=180n
CT1794 t1794 0 0.1f
M4747 t1791 nw478 t1794 0 nch w=1u l=180n
M4748 t1794 nq61 0 0 nch w=1u l=180n
M4749 t1792 nw478 vdd vdd pch w=2u l=180n
M4750 t1792 t1791 vdd vdd pch w=2u l=180n
CT1795 t1795 0 0.1f
M4751 t1792 nw478 t1795 0 nch w=1u l=180n
M4752 t1795 t1791 0 0 nch w=1u l=180n
M4753 t1793 nq61 vdd vdd pch w=2u l=180n
M4754 t1793 t1791 vdd vdd pch w=2u l=180n
CT1796 t1796 0 0.1f
M4755 t1793 nq61 t1796 0 nch w=1u l=180n
M4756 t1796 t1791 0 0 nch w=1u l=180n
M4757 nw583 t1792 vdd vdd pch w=2u l=180n
M4758 nw583 t1793 vdd vdd pch w=2u l=180n
CT1797 t1797 0 0.1f
M4759 nw583 t1792 t1797 0 nch w=1u l=180n
M4760 t1797 t1793 0 0 nch w=1u l=180n
Cnw583 nw583 0 2f
M4761 nw584 nw480 vdd vdd pch w=2u l=180n
M4762 nw584 nq63 vdd vdd pch w=2u l=180n
CT1798 t1798 0 0.1f
M4763 nw584 nw480 t1798 0 nch w=1u l=180n
M4764 t1798 nq63 0 0 nch w=1u l=180n
Cnw584 nw584 0 2f
M4765 nw585 nw482 0 0 nch w=1u l=180n
M4766 nw585 nq65 0 0 nch w=1u l=180n
CT1799 t1799 0 0.1f
M4767 t1799 nw482 vdd vdd pch w=2u l=180n
M4768 nw585 nq65 t1799 vdd pch w=2u l=180n
Cnw585 nw585 0 2f
CT1800 t1800 0 0.1f
M4769 t1800 nw484 vdd vdd pch w=2u l=180n
M4770 t1800 nq67 vdd vdd pch w=2u l=180n
CT1801 t1801 0 0.1f
M4771 t1800 nw484 t1801 0 nch w=1u l=180n
M4772 t1801 nq67 0 0 nch w=1u l=180n
M4773 nw586 t1800 vdd vdd pch w=2u l=180n
M4774 nw586 t1800 0 0 nch w=1u l=180n
Cnw586 nw586 0 2f
CT1802 t1802 0 0.1f
M4775 t1802 nw486 0 0 nch w=1u l=180n
M4776 t1802 nq69 0 0 nch w=1u l=180n
CT1803 t1803 0 0.1f
M4777 t1803 nw486 vdd vdd pch w=2u l=180n
M4778 t1802 nq69 t1803 vdd pch w=2u l=180n
M4779 nw587 t1802 vdd vdd pch w=2u l=180n
M4780 nw587 t1802 0 0 nch w=1u l=180n
Cnw587 nw587 0 2f
CT1804 t1804 0 0.1f
CT1805 t1805 0 0.1f
CT1806 t1806 0 0.1f
M4781 t1804 nw488 vdd vdd pch w=2u l=180n
M4782 t1804 nq71 vdd vdd pch w=2u l=180n
CT1807 t1807 0 0.1f
M4783 t1804 nw488 t1807 0 nch w=1u l=180n
M4784 t1807 nq71 0 0 nch w=1u l=180n
M4785 t1805 nw488 vdd vdd pch w=2u l=180n
M4786 t1805 t1804 vdd vdd pch w=2u l=180n
CT1808 t1808 0 0.1f
M4787 t1805 nw488 t1808 0 nch w=1u l=180n
M4788 t1808 t1804 0 0 nch w=1u l=180n
M4789 t1806 nq71 vdd vdd pch w=2u l=180n
M4790 t1806 t1804 vdd vdd pch w=2u l=180n
CT1809 t1809 0 0.1f
M4791 t1806 nq71 t1809 0 nch w=1u l=180n
M4792 t1809 t1804 0 0 nch w=1u l=180n
M4793 nw588 t1805 vdd vdd pch w=2u l=180n
M4794 nw588 t1806 vdd vdd pch w=2u l=180n
CT1810 t1810 0 0.1f
M4795 nw588 t1805 t1810 0 nch w=1u l=180n
M4796 t1810 t1806 0 0 nch w=1u l=180n
Cnw588 nw588 0 2f
M4797 nw589 nw490 vdd vdd pch w=2u l=180n
M4798 nw589 nq73 vdd vdd pch w=2u l=180n
CT1811 t1811 0 0.1f
M4799 nw589 nw490 t1811 0 nch w=1u l=180n
M4800 t1811 nq73 0 0 nch w=1u l=180n
Cnw589 nw589 0 2f
M4801 nw590 nw492 0 0 nch w=1u l=180n
M4802 nw590 ni1 0 0 nch w=1u l=180n
CT1812 t1812 0 0.1f
M4803 t1812 nw492 vdd vdd pch w=2u l=180n
M4804 nw590 ni1 t1812 vdd pch w=2u l=180n
Cnw590 nw590 0 2f
CT1813 t1813 0 0.1f
M4805 t1813 nw494 vdd vdd pch w=2u l=180n
M4806 t1813 ni3 vdd vdd pch w=2u l=180n
CT1814 t1814 0 0.1f
M4807 t1813 nw494 t1814 0 nch w=1u l=180n
M4808 t1814 ni3 0 0 nch w=1u l=180n
M4809 nw591 t1813 vdd vdd pch w=2u l=180n
M4810 nw591 t1813 0 0 nch w=1u l=180n
Cnw591 nw591 0 2f
CT1815 t1815 0 0.1f
M4811 t1815 nw496 0 0 nch w=1u l=180n
M4812 t1815 ni5 0 0 nch w=1u l=180n
CT1816 t1816 0 0.1f
M4813 t1816 nw496 vdd vdd pch w=2u l=180n
M4814 t1815 ni5 t1816 vdd pch w=2u l=180n
M4815 nw592 t1815 vdd vdd pch w=2u l=180n
M4816 nw592 t1815 0 0 nch w=1u l=180n
Cnw592 nw592 0 2f
CT1817 t1817 0 0.1f
CT1818 t1818 0 0.1f
CT1819 t1819 0 0.1f
M4817 t1817 nw498 vdd vdd pch w=2u l=180n
M4818 t1817 ni7 vdd vdd pch w=2u l=180n
CT1820 t1820 0 0.1f
M4819 t1817 nw498 t1820 0 nch w=1u l=180n
M4820 t1820 ni7 0 0 nch w=1u l=180n
M4821 t1818 nw498 vdd vdd pch w=2u l=180n
M4822 t1818 t1817 vdd vdd pch w=2u l=180n
CT1821 t1821 0 0.1f
M4823 t1818 nw498 t1821 0 nch w=1u l=180n
M4824 t1821 t1817 0 0 nch w=1u l=180n
M4825 t1819 ni7 vdd vdd pch w=2u l=180n
M4826 t1819 t1817 vdd vdd pch w=2u l=180n
CT1822 t1822 0 0.1f
M4827 t1819 ni7 t1822 0 nch w=1u l=180n
M4828 t1822 t1817 0 0 nch w=1u l=180n
M4829 nw593 t1818 vdd vdd pch w=2u l=180n
M4830 nw593 t1819 vdd vdd pch w=2u l=180n
CT1823 t1823 0 0.1f
M4831 nw593 t1818 t1823 0 nch w=1u l=180n
M4832 t1823 t1819 0 0 nch w=1u l=180n
Cnw593 nw593 0 2f
M4833 nw594 nw500 vdd vdd pch w=2u l=180n
M4834 nw594 ni9 vdd vdd pch w=2u l=180n
CT1824 t1824 0 0.1f
M4835 nw594 nw500 t1824 0 nch w=1u l=180n
M4836 t1824 ni9 0 0 nch w=1u l=180n
Cnw594 nw594 0 2f
M4837 nw595 nw502 0 0 nch w=1u l=180n
M4838 nw595 ni11 0 0 nch w=1u l=180n
CT1825 t1825 0 0.1f
M4839 t1825 nw502 vdd vdd pch w=2u l=180n
M4840 nw595 ni11 t1825 vdd pch w=2u l=180n
Cnw595 nw595 0 2f
CT1826 t1826 0 0.1f
M4841 t1826 nw504 vdd vdd pch w=2u l=180n
M4842 t1826 ni13 vdd vdd pch w=2u l=180n
CT1827 t1827 0 0.1f
M4843 t1826 nw504 t1827 0 nch w=1u l=180n
M4844 t1827 ni13 0 0 nch w=1u l=180n
M4845 nw596 t1826 vdd vdd pch w=2u l=180n
M4846 nw596 t1826 0 0 nch w=1u l=180n
Cnw596 nw596 0 2f
CT1828 t1828 0 0.1f
M4847 t1828 nw506 0 0 nch w=1u l=180n
M4848 t1828 ni15 0 0 nch w=1u l=180n
CT1829 t1829 0 0.1f
M4849 t1829 nw506 vdd vdd pch w=2u l=180n
M4850 t1828 ni15 t1829 vdd pch w=2u l=180n
M4851 nw597 t1828 vdd vdd pch w=2u l=180n
M4852 nw597 t1828 0 0 nch w=1u l=180n
Cnw597 nw597 0 2f
CT1830 t1830 0 0.1f
CT1831 t1831 0 0.1f
CT1832 t1832 0 0.1f
M4853 t1830 nw508 vdd vdd pch w=2u l=180n
M4854 t1830 nw150 vdd vdd pch w=2u l=180n
CT1833 t1833 0 0.1f
M4855 t1830 nw508 t1833 0 nch w=1u l=180n
M4856 t1833 nw150 0 0 nch w=1u l=180n
M4857 t1831 nw508 vdd vdd pch w=2u l=180n
M4858 t1831 t1830 vdd vdd pch w=2u l=180n
CT1834 t1834 0 0.1f
M4859 t1831 nw508 t1834 0 nch w=1u l=180n
M4860 t1834 t1830 0 0 nch w=1u l=180n
M4861 t1832 nw150 vdd vdd pch w=2u l=180n
M4862 t1832 t1830 vdd vdd pch w=2u l=180n
CT1835 t1835 0 0.1f
M4863 t1832 nw150 t1835 0 nch w=1u l=180n
M4864 t1835 t1830 0 0 nch w=1u l=180n
M4865 nw598 t1831 vdd vdd pch w=2u l=180n
M4866 nw598 t1832 vdd vdd pch w=2u l=180n
CT1836 t1836 0 0.1f
M4867 nw598 t1831 t1836 0 nch w=1u l=180n
M4868 t1836 t1832 0 0 nch w=1u l=180n
Cnw598 nw598 0 2f
M4869 nw599 nw510 vdd vdd pch w=2u l=180n
M4870 nw599 nw152 vdd vdd pch w=2u l=180n
CT1837 t1837 0 0.1f
M4871 nw599 nw510 t1837 0 nch w=1u l=180n
M4872 t1837 nw152 0 0 nch w=1u l=180n
Cnw599 nw599 0 2f
M4873 nw600 nw512 0 0 nch w=1u l=180n
M4874 nw600 nw154 0 0 nch w=1u l=180n
CT1838 t1838 0 0.1f
M4875 t1838 nw512 vdd vdd pch w=2u l=180n
M4876 nw600 nw154 t1838 vdd pch w=2u l=180n
Cnw600 nw600 0 2f
CT1839 t1839 0 0.1f
M4877 t1839 nw514 vdd vdd pch w=2u l=180n
M4878 t1839 nw156 vdd vdd pch w=2u l=180n
CT1840 t1840 0 0.1f
M4879 t1839 nw514 t1840 0 nch w=1u l=180n
M4880 t1840 nw156 0 0 nch w=1u l=180n
M4881 nw601 t1839 vdd vdd pch w=2u l=180n
M4882 nw601 t1839 0 0 nch w=1u l=180n
Cnw601 nw601 0 2f
CT1841 t1841 0 0.1f
M4883 t1841 nw516 0 0 nch w=1u l=180n
M4884 t1841 nw158 0 0 nch w=1u l=180n
CT1842 t1842 0 0.1f
M4885 t1842 nw516 vdd vdd pch w=2u l=180n
M4886 t1841 nw158 t1842 vdd pch w=2u l=180n
M4887 nw602 t1841 vdd vdd pch w=2u l=180n
M4888 nw602 t1841 0 0 nch w=1u l=180n
Cnw602 nw602 0 2f
CT1843 t1843 0 0.1f
CT1844 t1844 0 0.1f
CT1845 t1845 0 0.1f
M4889 t1843 nw518 vdd vdd pch w=2u l=180n
M4890 t1843 nw160 vdd vdd pch w=2u l=180n
CT1846 t1846 0 0.1f
M4891 t1843 nw518 t1846 0 nch w=1u l=180n
M4892 t1846 nw160 0 0 nch w=1u l=180n
M4893 t1844 nw518 vdd vdd pch w=2u l=180n
M4894 t1844 t1843 vdd vdd pch w=2u l=180n
CT1847 t1847 0 0.1f
M4895 t1844 nw518 t1847 0 nch w=1u l=180n
M4896 t1847 t1843 0 0 nch w=1u l=180n
M4897 t1845 nw160 vdd vdd pch w=2u l=180n
M4898 t1845 t1843 vdd vdd pch w=2u l=180n
CT1848 t1848 0 0.1f
M4899 t1845 nw160 t1848 0 nch w=1u l=180n
M4900 t1848 t1843 0 0 nch w=1u l=180n
M4901 nw603 t1844 vdd vdd pch w=2u l=180n
M4902 nw603 t1845 vdd vdd pch w=2u l=180n
CT1849 t1849 0 0.1f
M4903 nw603 t1844 t1849 0 nch w=1u l=180n
M4904 t1849 t1845 0 0 nch w=1u l=180n
Cnw603 nw603 0 2f
M4905 nw604 nw520 vdd vdd pch w=2u l=180n
M4906 nw604 nw162 vdd vdd pch w=2u l=180n
CT1850 t1850 0 0.1f
M4907 nw604 nw520 t1850 0 nch w=1u l=180n
M4908 t1850 nw162 0 0 nch w=1u l=180n
Cnw604 nw604 0 2f
M4909 nw605 nw522 0 0 nch w=1u l=180n
M4910 nw605 nw164 0 0 nch w=1u l=180n
CT1851 t1851 0 0.1f
M4911 t1851 nw522 vdd vdd pch w=2u l=180n
M4912 nw605 nw164 t1851 vdd pch w=2u l=180n
Cnw605 nw605 0 2f
CT1852 t1852 0 0.1f
M4913 t1852 nw524 vdd vdd pch w=2u l=180n
M4914 t1852 nw166 vdd vdd pch w=2u l=180n
CT1853 t1853 0 0.1f
M4915 t1852 nw524 t1853 0 nch w=1u l=180n
M4916 t1853 nw166 0 0 nch w=1u l=180n
M4917 nw606 t1852 vdd vdd pch w=2u l=180n
M4918 nw606 t1852 0 0 nch w=1u l=180n
Cnw606 nw606 0 2f
CT1854 t1854 0 0.1f
M4919 t1854 nw526 0 0 nch w=1u l=180n
M4920 t1854 nw168 0 0 nch w=1u l=180n
CT1855 t1855 0 0.1f
M4921 t1855 nw526 vdd vdd pch w=2u l=180n
M4922 t1854 nw168 t1855 vdd pch w=2u l=180n
M4923 nw607 t1854 vdd vdd pch w=2u l=180n
M4924 nw607 t1854 0 0 nch w=1u l=180n
Cnw607 nw607 0 2f
CT1856 t1856 0 0.1f
CT1857 t1857 0 0.1f
CT1858 t1858 0 0.1f
M4925 t1856 nw528 vdd vdd pch w=2u l=180n
M4926 t1856 nw170 vdd vdd pch w=2u l=180n
CT1859 t1859 0 0.1f
M4927 t1856 nw528 t1859 0 nch w=1u l=180n
M4928 t1859 nw170 0 0 nch w=1u l=180n
M4929 t1857 nw528 vdd vdd pch w=2u l=180n
M4930 t1857 t1856 vdd vdd pch w=2u l=180n
CT1860 t1860 0 0.1f
M4931 t1857 nw528 t1860 0 nch w=1u l=180n
M4932 t1860 t1856 0 0 nch w=1u l=180n
M4933 t1858 nw170 vdd vdd pch w=2u l=180n
M4934 t1858 t1856 vdd vdd pch w=2u l=180n
CT1861 t1861 0 0.1f
M4935 t1858 nw170 t1861 0 nch w=1u l=180n
M4936 t1861 t1856 0 0 nch w=1u l=180n
M4937 nw608 t1857 vdd vdd pch w=2u l=180n
M4938 nw608 t1858 vdd vdd pch w=2u l=180n
CT1862 t1862 0 0.1f
M4939 nw608 t1857 t1862 0 nch w=1u l=180n
M4940 t1862 t1858 0 0 nch w=1u l=180n
Cnw608 nw608 0 2f
M4941 nw609 nw530 vdd vdd pch w=2u l=180n
M4942 nw609 nw172 vdd vdd pch w=2u l=180n
CT1863 t1863 0 0.1f
M4943 nw609 nw530 t1863 0 nch w=1u l=180n
M4944 t1863 nw172 0 0 nch w=1u l=180n
Cnw609 nw609 0 2f
M4945 nw610 nw532 0 0 nch w=1u l=180n
M4946 nw610 nw174 0 0 nch w=1u l=180n
CT1864 t1864 0 0.1f
M4947 t1864 nw532 vdd vdd pch w=2u l=180n
M4948 nw610 nw174 t1864 vdd pch w=2u l=180n
Cnw610 nw610 0 2f
CT1865 t1865 0 0.1f
M4949 t1865 nw534 vdd vdd pch w=2u l=180n
M4950 t1865 nw176 vdd vdd pch w=2u l=180n
CT1866 t1866 0 0.1f
M4951 t1865 nw534 t1866 0 nch w=1u l=180n
M4952 t1866 nw176 0 0 nch w=1u l=180n
M4953 nw611 t1865 vdd vdd pch w=2u l=180n
M4954 nw611 t1865 0 0 nch w=1u l=180n
Cnw611 nw611 0 2f
CT1867 t1867 0 0.1f
M4955 t1867 nw536 0 0 nch w=1u l=180n
M4956 t1867 nw178 0 0 nch w=1u l=180n
CT1868 t1868 0 0.1f
M4957 t1868 nw536 vdd vdd pch w=2u l=180n
M4958 t1867 nw178 t1868 vdd pch w=2u l=180n
M4959 nw612 t1867 vdd vdd pch w=2u l=180n
M4960 nw612 t1867 0 0 nch w=1u l=180n
Cnw612 nw612 0 2f
CT1869 t1869 0 0.1f
CT1870 t1870 0 0.1f
CT1871 t1871 0 0.1f
M4961 t1869 nw538 vdd vdd pch w=2u l=180n
M4962 t1869 nw180 vdd vdd pch w=2u l=180n
CT1872 t1872 0 0.1f
M4963 t1869 nw538 t1872 0 nch w=1u l=180n
M4964 t1872 nw180 0 0 nch w=1u l=180n
M4965 t1870 nw538 vdd vdd pch w=2u l=180n
M4966 t1870 t1869 vdd vdd pch w=2u l=180n
CT1873 t1873 0 0.1f
M4967 t1870 nw538 t1873 0 nch w=1u l=180n
M4968 t1873 t1869 0 0 nch w=1u l=180n
M4969 t1871 nw180 vdd vdd pch w=2u l=180n
M4970 t1871 t1869 vdd vdd pch w=2u l=180n
CT1874 t1874 0 0.1f
M4971 t1871 nw180 t1874 0 nch w=1u l=180n
M4972 t1874 t1869 0 0 nch w=1u l=180n
M4973 nw613 t1870 vdd vdd pch w=2u l=180n
M4974 nw613 t1871 vdd vdd pch w=2u l=180n
CT1875 t1875 0 0.1f
M4975 nw613 t1870 t1875 0 nch w=1u l=180n
M4976 t1875 t1871 0 0 nch w=1u l=180n
Cnw613 nw613 0 2f
M4977 nw614 nw540 vdd vdd pch w=2u l=180n
M4978 nw614 nw182 vdd vdd pch w=2u l=180n
CT1876 t1876 0 0.1f
M4979 nw614 nw540 t1876 0 nch w=1u l=180n
M4980 t1876 nw182 0 0 nch w=1u l=180n
Cnw614 nw614 0 2f
M4981 nw615 nw542 0 0 nch w=1u l=180n
M4982 nw615 nw184 0 0 nch w=1u l=180n
CT1877 t1877 0 0.1f
M4983 t1877 nw542 vdd vdd pch w=2u l=180n
M4984 nw615 nw184 t1877 vdd pch w=2u l=180n
Cnw615 nw615 0 2f
CT1878 t1878 0 0.1f
M4985 t1878 nw544 vdd vdd pch w=2u l=180n
M4986 t1878 nw186 vdd vdd pch w=2u l=180n
CT1879 t1879 0 0.1f
M4987 t1878 nw544 t1879 0 nch w=1u l=180n
M4988 t1879 nw186 0 0 nch w=1u l=180n
M4989 nw616 t1878 vdd vdd pch w=2u l=180n
M4990 nw616 t1878 0 0 nch w=1u l=180n
Cnw616 nw616 0 2f
CT1880 t1880 0 0.1f
M4991 t1880 nw546 0 0 nch w=1u l=180n
M4992 t1880 nw188 0 0 nch w=1u l=180n
CT1881 t1881 0 0.1f
M4993 t1881 nw546 vdd vdd pch w=2u l=180n
M4994 t1880 nw188 t1881 vdd pch w=2u l=180n
M4995 nw617 t1880 vdd vdd pch w=2u l=180n
M4996 nw617 t1880 0 0 nch w=1u l=180n
Cnw617 nw617 0 2f
CT1882 t1882 0 0.1f
CT1883 t1883 0 0.1f
CT1884 t1884 0 0.1f
M4997 t1882 nw548 vdd vdd pch w=2u l=180n
M4998 t1882 nw190 vdd vdd pch w=2u l=180n
CT1885 t1885 0 0.1f
M4999 t1882 nw548 t1885 0 nch w=1u l=180n
M5000 t1885 nw190 0 0 nch w=1u l=180n
M5001 t1883 nw548 vdd vdd pch w=2u l=180n
M5002 t1883 t1882 vdd vdd pch w=2u l=180n
CT1886 t1886 0 0.1f
M5003 t1883 nw548 t1886 0 nch w=1u l=180n
M5004 t1886 t1882 0 0 nch w=1u l=180n
M5005 t1884 nw190 vdd vdd pch w=2u l=180n
M5006 t1884 t1882 vdd vdd pch w=2u l=180n
CT1887 t1887 0 0.1f
M5007 t1884 nw190 t1887 0 nch w=1u l=180n
M5008 t1887 t1882 0 0 nch w=1u l=180n
M5009 nw618 t1883 vdd vdd pch w=2u l=180n
M5010 nw618 t1884 vdd vdd pch w=2u l=180n
CT1888 t1888 0 0.1f
M5011 nw618 t1883 t1888 0 nch w=1u l=180n
M5012 t1888 t1884 0 0 nch w=1u l=180n
Cnw618 nw618 0 2f
M5013 nw619 nw550 vdd vdd pch w=2u l=180n
M5014 nw619 nw192 vdd vdd pch w=2u l=180n
CT1889 t1889 0 0.1f
M5015 nw619 nw550 t1889 0 nch w=1u l=180n
M5016 t1889 nw192 0 0 nch w=1u l=180n
Cnw619 nw619 0 2f
M5017 nw620 nw552 0 0 nch w=1u l=180n
M5018 nw620 nw194 0 0 nch w=1u l=180n
CT1890 t1890 0 0.1f
M5019 t1890 nw552 vdd vdd pch w=2u l=180n
M5020 nw620 nw194 t1890 vdd pch w=2u l=180n
Cnw620 nw620 0 2f
CT1891 t1891 0 0.1f
M5021 t1891 nw554 vdd vdd pch w=2u l=180n
M5022 t1891 nw196 vdd vdd pch w=2u l=180n
CT1892 t1892 0 0.1f
M5023 t1891 nw554 t1892 0 nch w=1u l=180n
M5024 t1892 nw196 0 0 nch w=1u l=180n
M5025 nw621 t1891 vdd vdd pch w=2u l=180n
M5026 nw621 t1891 0 0 nch w=1u l=180n
Cnw621 nw621 0 2f
CT1893 t1893 0 0.1f
M5027 t1893 nw556 0 0 nch w=1u l=180n
M5028 t1893 nw198 0 0 nch w=1u l=180n
CT1894 t1894 0 0.1f
M5029 t1894 nw556 vdd vdd pch w=2u l=180n
M5030 t1893 nw198 t1894 vdd pch w=2u l=180n
M5031 nw622 t1893 vdd vdd pch w=2u l=180n
M5032 nw622 t1893 0 0 nch w=1u l=180n
Cnw622 nw622 0 2f
CT1895 t1895 0 0.1f
CT1896 t1896 0 0.1f
CT1897 t1897 0 0.1f
M5033 t1895 nw558 vdd vdd pch w=2u l=180n
M5034 t1895 nw200 vdd vdd pch w=2u l=180n
CT1898 t1898 0 0.1f
M5035 t1895 nw558 t1898 0 nch w=1u l=180n
M5036 t1898 nw200 0 0 nch w=1u l=180n
M5037 t1896 nw558 vdd vdd pch w=2u l=180n
M5038 t1896 t1895 vdd vdd pch w=2u l=180n
CT1899 t1899 0 0.1f
M5039 t1896 nw558 t1899 0 nch w=1u l=180n
M5040 t1899 t1895 0 0 nch w=1u l=180n
M5041 t1897 nw200 vdd vdd pch w=2u l=180n
M5042 t1897 t1895 vdd vdd pch w=2u l=180n
CT1900 t1900 0 0.1f
M5043 t1897 nw200 t1900 0 nch w=1u l=180n
M5044 t1900 t1895 0 0 nch w=1u l=180n
M5045 nw623 t1896 vdd vdd pch w=2u l=180n
M5046 nw623 t1897 vdd vdd pch w=2u l=180n
CT1901 t1901 0 0.1f
M5047 nw623 t1896 t1901 0 nch w=1u l=180n
M5048 t1901 t1897 0 0 nch w=1u l=180n
Cnw623 nw623 0 2f
M5049 nw624 nw560 vdd vdd pch w=2u l=180n
M5050 nw624 nw202 vdd vdd pch w=2u l=180n
CT1902 t1902 0 0.1f
M5051 nw624 nw560 t1902 0 nch w=1u l=180n
M5052 t1902 nw202 0 0 nch w=1u l=180n
Cnw624 nw624 0 2f
M5053 nw625 nw562 0 0 nch w=1u l=180n
M5054 nw625 nw204 0 0 nch w=1u l=180n
CT1903 t1903 0 0.1f
M5055 t1903 nw562 vdd vdd pch w=2u l=180n
M5056 nw625 nw204 t1903 vdd pch w=2u l=180n
Cnw625 nw625 0 2f
CT1904 t1904 0 0.1f
M5057 t1904 nw564 vdd vdd pch w=2u l=180n
M5058 t1904 nw206 vdd vdd pch w=2u l=180n
CT1905 t1905 0 0.1f
M5059 t1904 nw564 t1905 0 nch w=1u l=180n
M5060 t1905 nw206 0 0 nch w=1u l=180n
M5061 nw626 t1904 vdd vdd pch w=2u l=180n
M5062 nw626 t1904 0 0 nch w=1u l=180n
Cnw626 nw626 0 2f
CT1906 t1906 0 0.1f
M5063 t1906 nw566 0 0 nch w=1u l=180n
M5064 t1906 nw208 0 0 nch w=1u l=180n
CT1907 t1907 0 0.1f
M5065 t1907 nw566 vdd vdd pch w=2u l=180n
M5066 t1906 nw208 t1907 vdd pch w=2u l=180n
M5067 nw627 t1906 vdd vdd pch w=2u l=180n
M5068 nw627 t1906 0 0 nch w=1u l=180n
Cnw627 nw627 0 2f
CT1908 t1908 0 0.1f
CT1909 t1909 0 0.1f
CT1910 t1910 0 0.1f
M5069 t1908 nw568 vdd vdd pch w=2u l=180n
M5070 t1908 nw210 vdd vdd pch w=2u l=180n
CT1911 t1911 0 0.1f
M5071 t1908 nw568 t1911 0 nch w=1u l=180n
M5072 t1911 nw210 0 0 nch w=1u l=180n
M5073 t1909 nw568 vdd vdd pch w=2u l=180n
M5074 t1909 t1908 vdd vdd pch w=2u l=180n
CT1912 t1912 0 0.1f
M5075 t1909 nw568 t1912 0 nch w=1u l=180n
M5076 t1912 t1908 0 0 nch w=1u l=180n
M5077 t1910 nw210 vdd vdd pch w=2u l=180n
M5078 t1910 t1908 vdd vdd pch w=2u l=180n
CT1913 t1913 0 0.1f
M5079 t1910 nw210 t1913 0 nch w=1u l=180n
M5080 t1913 t1908 0 0 nch w=1u l=180n
M5081 nw628 t1909 vdd vdd pch w=2u l=180n
M5082 nw628 t1910 vdd vdd pch w=2u l=180n
CT1914 t1914 0 0.1f
M5083 nw628 t1909 t1914 0 nch w=1u l=180n
M5084 t1914 t1910 0 0 nch w=1u l=180n
Cnw628 nw628 0 2f
M5085 nw629 nw570 vdd vdd pch w=2u l=180n
M5086 nw629 nw212 vdd vdd pch w=2u l=180n
CT1915 t1915 0 0.1f
M5087 nw629 nw570 t1915 0 nch w=1u l=180n
M5088 t1915 nw212 0 0 nch w=1u l=180n
Cnw629 nw629 0 2f
M5089 nw630 nw572 0 0 nch w=1u l=180n
M5090 nw630 nw214 0 0 nch w=1u l=180n
CT1916 t1916 0 0.1f
M5091 t1916 nw572 vdd vdd pch w=2u l=180n
M5092 nw630 nw214 t1916 vdd pch w=2u l=180n
Cnw630 nw630 0 2f
CT1917 t1917 0 0.1f
M5093 t1917 nw574 vdd vdd pch w=2u l=180n
M5094 t1917 nw216 vdd vdd pch w=2u l=180n
CT1918 t1918 0 0.1f
M5095 t1917 nw574 t1918 0 nch w=1u l=180n
M5096 t1918 nw216 0 0 nch w=1u l=180n
M5097 nw631 t1917 vdd vdd pch w=2u l=180n
M5098 nw631 t1917 0 0 nch w=1u l=180n
Cnw631 nw631 0 2f
CT1919 t1919 0 0.1f
M5099 t1919 nw576 0 0 nch w=1u l=180n
M5100 t1919 nw218 0 0 nch w=1u l=180n
CT1920 t1920 0 0.1f
M5101 t1920 nw576 vdd vdd pch w=2u l=180n
M5102 t1919 nw218 t1920 vdd pch w=2u l=180n
M5103 nw632 t1919 vdd vdd pch w=2u l=180n
M5104 nw632 t1919 0 0 nch w=1u l=180n
Cnw632 nw632 0 2f
CT1921 t1921 0 0.1f
CT1922 t1922 0 0.1f
CT1923 t1923 0 0.1f
M5105 t1921 nw578 vdd vdd pch w=2u l=180n
M5106 t1921 nw220 vdd vdd pch w=2u l=180n
CT1924 t1924 0 0.1f
M5107 t1921 nw578 t1924 0 nch w=1u l=180n
M5108 t1924 nw220 0 0 nch w=1u l=180n
M5109 t1922 nw578 vdd vdd pch w=2u l=180n
M5110 t1922 t1921 vdd vdd pch w=2u l=180n
CT1925 t1925 0 0.1f
M5111 t1922 nw578 t1925 0 nch w=1u l=180n
M5112 t1925 t1921 0 0 nch w=1u l=180n
M5113 t1923 nw220 vdd vdd pch w=2u l=180n
M5114 t1923 t1921 vdd vdd pch w=2u l=180n
CT1926 t1926 0 0.1f
M5115 t1923 nw220 t1926 0 nch w=1u l=180n
M5116 t1926 t1921 0 0 nch w=1u l=180n
M5117 nw633 t1922 vdd vdd pch w=2u l=180n
M5118 nw633 t1923 vdd vdd pch w=2u l=180n
CT1927 t1927 0 0.1f
M5119 nw633 t1922 t1927 0 nch w=1u l=180n
M5120 t1927 t1923 0 0 nch w=1u l=180n
Cnw633 nw633 0 2f
M5121 nw634 nw580 vdd vdd pch w=2u l=180n
M5122 nw634 nw222 vdd vdd pch w=2u l=180n
CT1928 t1928 0 0.1f
M5123 nw634 nw580 t1928 0 nch w=1u l=180n
M5124 t1928 nw222 0 0 nch w=1u l=180n
Cnw634 nw634 0 2f
M5125 nw635 nw582 0 0 nch w=1u l=180n
M5126 nw635 nw224 0 0 nch w=1u l=180n
CT1929 t1929 0 0.1f
M5127 t1929 nw582 vdd vdd pch w=2u l=180n
M5128 nw635 nw224 t1929 vdd pch w=2u l=180n
Cnw635 nw635 0 2f
CT1930 t1930 0 0.1f
M5129 t1930 nw584 vdd vdd pch w=2u l=180n
M5130 t1930 nw226 vdd vdd pch w=2u l=180n
CT1931 t1931 0 0.1f
M5131 t1930 nw584 t1931 0 nch w=1u l=180n
M5132 t1931 nw226 0 0 nch w=1u l=180n
M5133 nw636 t1930 vdd vdd pch w=2u l=180n
M5134 nw636 t1930 0 0 nch w=1u l=180n
Cnw636 nw636 0 2f
CT1932 t1932 0 0.1f
M5135 t1932 nw586 0 0 nch w=1u l=180n
M5136 t1932 nw228 0 0 nch w=1u l=180n
CT1933 t1933 0 0.1f
M5137 t1933 nw586 vdd vdd pch w=2u l=180n
M5138 t1932 nw228 t1933 vdd pch w=2u l=180n
M5139 nw637 t1932 vdd vdd pch w=2u l=180n
M5140 nw637 t1932 0 0 nch w=1u l=180n
Cnw637 nw637 0 2f
CT1934 t1934 0 0.1f
CT1935 t1935 0 0.1f
CT1936 t1936 0 0.1f
M5141 t1934 nw588 vdd vdd pch w=2u l=180n
M5142 t1934 nw230 vdd vdd pch w=2u l=180n
CT1937 t1937 0 0.1f
M5143 t1934 nw588 t1937 0 nch w=1u l=180n
M5144 t1937 nw230 0 0 nch w=1u l=180n
M5145 t1935 nw588 vdd vdd pch w=2u l=180n
M5146 t1935 t1934 vdd vdd pch w=2u l=180n
CT1938 t1938 0 0.1f
M5147 t1935 nw588 t1938 0 nch w=1u l=180n
M5148 t1938 t1934 0 0 nch w=1u l=180n
M5149 t1936 nw230 vdd vdd pch w=2u l=180n
M5150 t1936 t1934 vdd vdd pch w=2u l=180n
CT1939 t1939 0 0.1f
M5151 t1936 nw230 t1939 0 nch w=1u l=180n
M5152 t1939 t1934 0 0 nch w=1u l=180n
M5153 nw638 t1935 vdd vdd pch w=2u l=180n
M5154 nw638 t1936 vdd vdd pch w=2u l=180n
CT1940 t1940 0 0.1f
M5155 nw638 t1935 t1940 0 nch w=1u l=180n
M5156 t1940 t1936 0 0 nch w=1u l=180n
Cnw638 nw638 0 2f
M5157 nw639 nw590 vdd vdd pch w=2u l=180n
M5158 nw639 nw232 vdd vdd pch w=2u l=180n
CT1941 t1941 0 0.1f
M5159 nw639 nw590 t1941 0 nch w=1u l=180n
M5160 t1941 nw232 0 0 nch w=1u l=180n
Cnw639 nw639 0 2f
M5161 nw640 nw592 0 0 nch w=1u l=180n
M5162 nw640 nw234 0 0 nch w=1u l=180n
CT1942 t1942 0 0.1f
M5163 t1942 nw592 vdd vdd pch w=2u l=180n
M5164 nw640 nw234 t1942 vdd pch w=2u l=180n
Cnw640 nw640 0 2f
CT1943 t1943 0 0.1f
M5165 t1943 nw594 vdd vdd pch w=2u l=180n
M5166 t1943 nw236 vdd vdd pch w=2u l=180n
CT1944 t1944 0 0.1f
M5167 t1943 nw594 t1944 0 nch w=1u l=180n
M5168 t1944 nw236 0 0 nch w=1u l=180n
M5169 nw641 t1943 vdd vdd pch w=2u l=180n
M5170 nw641 t1943 0 0 nch w=1u l=180n
Cnw641 nw641 0 2f
CT1945 t1945 0 0.1f
M5171 t1945 nw596 0 0 nch w=1u l=180n
M5172 t1945 nw238 0 0 nch w=1u l=180n
CT1946 t1946 0 0.1f
M5173 t1946 nw596 vdd vdd pch w=2u l=180n
M5174 t1945 nw238 t1946 vdd pch w=2u l=180n
M5175 nw642 t1945 vdd vdd pch w=2u l=180n
M5176 nw642 t1945 0 0 nch w=1u l=180n
Cnw642 nw642 0 2f
CT1947 t1947 0 0.1f
CT1948 t1948 0 0.1f
CT1949 t1949 0 0.1f
M5177 t1947 nw598 vdd vdd pch w=2u l=180n
M5178 t1947 nw240 vdd vdd pch w=2u l=180n
CT1950 t1950 0 0.1f
M5179 t1947 nw598 t1950 0 nch w=1u l=180n
M5180 t1950 nw240 0 0 nch w=1u l=180n
M5181 t1948 nw598 vdd vdd pch w=2u l=180n
M5182 t1948 t1947 vdd vdd pch w=2u l=180n
CT1951 t1951 0 0.1f
M5183 t1948 nw598 t1951 0 nch w=1u l=180n
M5184 t1951 t1947 0 0 nch w=1u l=180n
M5185 t1949 nw240 vdd vdd pch w=2u l=180n
M5186 t1949 t1947 vdd vdd pch w=2u l=180n
CT1952 t1952 0 0.1f
M5187 t1949 nw240 t1952 0 nch w=1u l=180n
M5188 t1952 t1947 0 0 nch w=1u l=180n
M5189 nw643 t1948 vdd vdd pch w=2u l=180n
M5190 nw643 t1949 vdd vdd pch w=2u l=180n
CT1953 t1953 0 0.1f
M5191 nw643 t1948 t1953 0 nch w=1u l=180n
M5192 t1953 t1949 0 0 nch w=1u l=180n
Cnw643 nw643 0 2f
M5193 nw644 nw600 vdd vdd pch w=2u l=180n
M5194 nw644 nw242 vdd vdd pch w=2u l=180n
CT1954 t1954 0 0.1f
M5195 nw644 nw600 t1954 0 nch w=1u l=180n
M5196 t1954 nw242 0 0 nch w=1u l=180n
Cnw644 nw644 0 2f
M5197 nw645 nw602 0 0 nch w=1u l=180n
M5198 nw645 nw244 0 0 nch w=1u l=180n
CT1955 t1955 0 0.1f
M5199 t1955 nw602 vdd vdd pch w=2u l=180n
M5200 nw645 nw244 t1955 vdd pch w=2u l=180n
Cnw645 nw645 0 2f
CT1956 t1956 0 0.1f
M5201 t1956 nw604 vdd vdd pch w=2u l=180n
M5202 t1956 nw246 vdd vdd pch w=2u l=180n
CT1957 t1957 0 0.1f
M5203 t1956 nw604 t1957 0 nch w=1u l=180n
M5204 t1957 nw246 0 0 nch w=1u l=180n
M5205 nw646 t1956 vdd vdd pch w=2u l=180n
M5206 nw646 t1956 0 0 nch w=1u l=180n
Cnw646 nw646 0 2f
CT1958 t1958 0 0.1f
M5207 t1958 nw606 0 0 nch w=1u l=180n
M5208 t1958 nw248 0 0 nch w=1u l=180n
CT1959 t1959 0 0.1f
M5209 t1959 nw606 vdd vdd pch w=2u l=180n
M5210 t1958 nw248 t1959 vdd pch w=2u l=180n
M5211 nw647 t1958 vdd vdd pch w=2u l=180n
M5212 nw647 t1958 0 0 nch w=1u l=180n
Cnw647 nw647 0 2f
CT1960 t1960 0 0.1f
CT1961 t1961 0 0.1f
CT1962 t1962 0 0.1f
M5213 t1960 nw608 vdd vdd pch w=2u l=180n
M5214 t1960 nw250 vdd vdd pch w=2u l=180n
CT1963 t1963 0 0.1f
M5215 t1960 nw608 t1963 0 nch w=1u l=180n
M5216 t1963 nw250 0 0 nch w=1u l=180n
M5217 t1961 nw608 vdd vdd pch w=2u l=180n
M5218 t1961 t1960 vdd vdd pch w=2u l=180n
CT1964 t1964 0 0.1f
M5219 t1961 nw608 t1964 0 nch w=1u l=180n
M5220 t1964 t1960 0 0 nch w=1u l=180n
M5221 t1962 nw250 vdd vdd pch w=2u l=180n
M5222 t1962 t1960 vdd vdd pch w=2u l=180n
CT1965 t1965 0 0.1f
M5223 t1962 nw250 t1965 0 nch w=1u l=180n
M5224 t1965 t1960 0 0 nch w=1u l=180n
M5225 nw648 t1961 vdd vdd pch w=2u l=180n
M5226 nw648 t1962 vdd vdd pch w=2u l=180n
CT1966 t1966 0 0.1f
M5227 nw648 t1961 t1966 0 nch w=1u l=180n
M5228 t1966 t1962 0 0 nch w=1u l=180n
Cnw648 nw648 0 2f
M5229 nw649 nw610 vdd vdd pch w=2u l=180n
M5230 nw649 nw252 vdd vdd pch w=2u l=180n
CT1967 t1967 0 0.1f
M5231 nw649 nw610 t1967 0 nch w=1u l=180n
M5232 t1967 nw252 0 0 nch w=1u l=180n
Cnw649 nw649 0 2f
M5233 nw650 nw612 0 0 nch w=1u l=180n
M5234 nw650 nw254 0 0 nch w=1u l=180n
CT1968 t1968 0 0.1f
M5235 t1968 nw612 vdd vdd pch w=2u l=180n
M5236 nw650 nw254 t1968 vdd pch w=2u l=180n
Cnw650 nw650 0 2f
CT1969 t1969 0 0.1f
M5237 t1969 nw614 vdd vdd pch w=2u l=180n
M5238 t1969 nw256 vdd vdd pch w=2u l=180n
CT1970 t1970 0 0.1f
M5239 t1969 nw614 t1970 0 nch w=1u l=180n
M5240 t1970 nw256 0 0 nch w=1u l=180n
M5241 nw651 t1969 vdd vdd pch w=2u l=180n
M5242 nw651 t1969 0 0 nch w=1u l=180n
Cnw651 nw651 0 2f
CT1971 t1971 0 0.1f
M5243 t1971 nw616 0 0 nch w=1u l=180n
M5244 t1971 nw258 0 0 nch w=1u l=180n
CT1972 t1972 0 0.1f
M5245 t1972 nw616 vdd vdd pch w=2u l=180n
M5246 t1971 nw258 t1972 vdd pch w=2u l=180n
M5247 nw652 t1971 vdd vdd pch w=2u l=180n
M5248 nw652 t1971 0 0 nch w=1u l=180n
Cnw652 nw652 0 2f
CT1973 t1973 0 0.1f
CT1974 t1974 0 0.1f
CT1975 t1975 0 0.1f
M5249 t1973 nw618 vdd vdd pch w=2u l=180n
M5250 t1973 nw260 vdd vdd pch w=2u l=180n
CT1976 t1976 0 0.1f
M5251 t1973 nw618 t1976 0 nch w=1u l=180n
M5252 t1976 nw260 0 0 nch w=1u l=180n
M5253 t1974 nw618 vdd vdd pch w=2u l=180n
M5254 t1974 t1973 vdd vdd pch w=2u l=180n
CT1977 t1977 0 0.1f
M5255 t1974 nw618 t1977 0 nch w=1u l=180n
M5256 t1977 t1973 0 0 nch w=1u l=180n
M5257 t1975 nw260 vdd vdd pch w=2u l=180n
M5258 t1975 t1973 vdd vdd pch w=2u l=180n
CT1978 t1978 0 0.1f
M5259 t1975 nw260 t1978 0 nch w=1u l=180n
M5260 t1978 t1973 0 0 nch w=1u l=180n
M5261 nw653 t1974 vdd vdd pch w=2u l=180n
M5262 nw653 t1975 vdd vdd pch w=2u l=180n
CT1979 t1979 0 0.1f
M5263 nw653 t1974 t1979 0 nch w=1u l=180n
M5264 t1979 t1975 0 0 nch w=1u l=180n
Cnw653 nw653 0 2f
M5265 nw654 nw620 vdd vdd pch w=2u l=180n
M5266 nw654 nw262 vdd vdd pch w=2u l=180n
CT1980 t1980 0 0.1f
M5267 nw654 nw620 t1980 0 nch w=1u l=180n
M5268 t1980 nw262 0 0 nch w=1u l=180n
Cnw654 nw654 0 2f
M5269 nw655 nw622 0 0 nch w=1u l=180n
M5270 nw655 nw264 0 0 nch w=1u l=180n
CT1981 t1981 0 0.1f
M5271 t1981 nw622 vdd vdd pch w=2u l=180n
M5272 nw655 nw264 t1981 vdd pch w=2u l=180n
Cnw655 nw655 0 2f
CT1982 t1982 0 0.1f
M5273 t1982 nw624 vdd vdd pch w=2u l=180n
M5274 t1982 nw266 vdd vdd pch w=2u l=180n
CT1983 t1983 0 0.1f
M5275 t1982 nw624 t1983 0 nch w=1u l=180n
M5276 t1983 nw266 0 0 nch w=1u l=180n
M5277 nw656 t1982 vdd vdd pch w=2u l=180n
M5278 nw656 t1982 0 0 nch w=1u l=180n
Cnw656 nw656 0 2f
CT1984 t1984 0 0.1f
M5279 t1984 nw626 0 0 nch w=1u l=180n
M5280 t1984 nw268 0 0 nch w=1u l=180n
CT1985 t1985 0 0.1f
M5281 t1985 nw626 vdd vdd pch w=2u l=180n
M5282 t1984 nw268 t1985 vdd pch w=2u l=180n
M5283 nw657 t1984 vdd vdd pch w=2u l=180n
M5284 nw657 t1984 0 0 nch w=1u l=180n
Cnw657 nw657 0 2f
CT1986 t1986 0 0.1f
CT1987 t1987 0 0.1f
CT1988 t1988 0 0.1f
M5285 t1986 nw628 vdd vdd pch w=2u l=180n
M5286 t1986 nw270 vdd vdd pch w=2u l=180n
CT1989 t1989 0 0.1f
M5287 t1986 nw628 t1989 0 nch w=1u l=180n
M5288 t1989 nw270 0 0 nch w=1u l=180n
M5289 t1987 nw628 vdd vdd pch w=2u l=180n
M5290 t1987 t1986 vdd vdd pch w=2u l=180n
CT1990 t1990 0 0.1f
M5291 t1987 nw628 t1990 0 nch w=1u l=180n
M5292 t1990 t1986 0 0 nch w=1u l=180n
M5293 t1988 nw270 vdd vdd pch w=2u l=180n
M5294 t1988 t1986 vdd vdd pch w=2u l=180n
CT1991 t1991 0 0.1f
M5295 t1988 nw270 t1991 0 nch w=1u l=180n
M5296 t1991 t1986 0 0 nch w=1u l=180n
M5297 nw658 t1987 vdd vdd pch w=2u l=180n
M5298 nw658 t1988 vdd vdd pch w=2u l=180n
CT1992 t1992 0 0.1f
M5299 nw658 t1987 t1992 0 nch w=1u l=180n
M5300 t1992 t1988 0 0 nch w=1u l=180n
Cnw658 nw658 0 2f
M5301 nw659 nw630 vdd vdd pch w=2u l=180n
M5302 nw659 nw272 vdd vdd pch w=2u l=180n
CT1993 t1993 0 0.1f
M5303 nw659 nw630 t1993 0 nch w=1u l=180n
M5304 t1993 nw272 0 0 nch w=1u l=180n
Cnw659 nw659 0 2f
M5305 nw660 nw632 0 0 nch w=1u l=180n
M5306 nw660 nw274 0 0 nch w=1u l=180n
CT1994 t1994 0 0.1f
M5307 t1994 nw632 vdd vdd pch w=2u l=180n
M5308 nw660 nw274 t1994 vdd pch w=2u l=180n
Cnw660 nw660 0 2f
CT1995 t1995 0 0.1f
M5309 t1995 nw634 vdd vdd pch w=2u l=180n
M5310 t1995 nw276 vdd vdd pch w=2u l=180n
CT1996 t1996 0 0.1f
M5311 t1995 nw634 t1996 0 nch w=1u l=180n
M5312 t1996 nw276 0 0 nch w=1u l=180n
M5313 nw661 t1995 vdd vdd pch w=2u l=180n
M5314 nw661 t1995 0 0 nch w=1u l=180n
Cnw661 nw661 0 2f
CT1997 t1997 0 0.1f
M5315 t1997 nw636 0 0 nch w=1u l=180n
M5316 t1997 nw278 0 0 nch w=1u l=180n
CT1998 t1998 0 0.1f
M5317 t1998 nw636 vdd vdd pch w=2u l=180n
M5318 t1997 nw278 t1998 vdd pch w=2u l=180n
M5319 nw662 t1997 vdd vdd pch w=2u l=180n
M5320 nw662 t1997 0 0 nch w=1u l=180n
Cnw662 nw662 0 2f
CT1999 t1999 0 0.1f
CT2000 t2000 0 0.1f
CT2001 t2001 0 0.1f
M5321 t1999 nw638 vdd vdd pch w=2u l=180n
M5322 t1999 nw280 vdd vdd pch w=2u l=180n
CT2002 t2002 0 0.1f
M5323 t1999 nw638 t2002 0 nch w=1u l=180n
M5324 t2002 nw280 0 0 nch w=1u l=180n
M5325 t2000 nw638 vdd vdd pch w=2u l=180n
M5326 t2000 t1999 vdd vdd pch w=2u l=180n
CT2003 t2003 0 0.1f
M5327 t2000 nw638 t2003 0 nch w=1u l=180n
M5328 t2003 t1999 0 0 nch w=1u l=180n
M5329 t2001 nw280 vdd vdd pch w=2u l=180n
M5330 t2001 t1999 vdd vdd pch w=2u l=180n
CT2004 t2004 0 0.1f
M5331 t2001 nw280 t2004 0 nch w=1u l=180n
M5332 t2004 t1999 0 0 nch w=1u l=180n
M5333 nw663 t2000 vdd vdd pch w=2u l=180n
M5334 nw663 t2001 vdd vdd pch w=2u l=180n
CT2005 t2005 0 0.1f
M5335 nw663 t2000 t2005 0 nch w=1u l=180n
M5336 t2005 t2001 0 0 nch w=1u l=180n
Cnw663 nw663 0 2f
M5337 nw664 nw640 vdd vdd pch w=2u l=180n
M5338 nw664 nw282 vdd vdd pch w=2u l=180n
CT2006 t2006 0 0.1f
M5339 nw664 nw640 t2006 0 nch w=1u l=180n
M5340 t2006 nw282 0 0 nch w=1u l=180n
Cnw664 nw664 0 2f
M5341 nw665 nw642 0 0 nch w=1u l=180n
M5342 nw665 nw284 0 0 nch w=1u l=180n
CT2007 t2007 0 0.1f
M5343 t2007 nw642 vdd vdd pch w=2u l=180n
M5344 nw665 nw284 t2007 vdd pch w=2u l=180n
Cnw665 nw665 0 2f
CT2008 t2008 0 0.1f
M5345 t2008 nw644 vdd vdd pch w=2u l=180n
M5346 t2008 nw286 vdd vdd pch w=2u l=180n
CT2009 t2009 0 0.1f
M5347 t2008 nw644 t2009 0 nch w=1u l=180n
M5348 t2009 nw286 0 0 nch w=1u l=180n
M5349 nw666 t2008 vdd vdd pch w=2u l=180n
M5350 nw666 t2008 0 0 nch w=1u l=180n
Cnw666 nw666 0 2f
CT2010 t2010 0 0.1f
M5351 t2010 nw646 0 0 nch w=1u l=180n
M5352 t2010 nw288 0 0 nch w=1u l=180n
CT2011 t2011 0 0.1f
M5353 t2011 nw646 vdd vdd pch w=2u l=180n
M5354 t2010 nw288 t2011 vdd pch w=2u l=180n
M5355 nw667 t2010 vdd vdd pch w=2u l=180n
M5356 nw667 t2010 0 0 nch w=1u l=180n
Cnw667 nw667 0 2f
CT2012 t2012 0 0.1f
CT2013 t2013 0 0.1f
CT2014 t2014 0 0.1f
M5357 t2012 nw648 vdd vdd pch w=2u l=180n
M5358 t2012 nw290 vdd vdd pch w=2u l=180n
CT2015 t2015 0 0.1f
M5359 t2012 nw648 t2015 0 nch w=1u l=180n
M5360 t2015 nw290 0 0 nch w=1u l=180n
M5361 t2013 nw648 vdd vdd pch w=2u l=180n
M5362 t2013 t2012 vdd vdd pch w=2u l=180n
CT2016 t2016 0 0.1f
M5363 t2013 nw648 t2016 0 nch w=1u l=180n
M5364 t2016 t2012 0 0 nch w=1u l=180n
M5365 t2014 nw290 vdd vdd pch w=2u l=180n
M5366 t2014 t2012 vdd vdd pch w=2u l=180n
CT2017 t2017 0 0.1f
M5367 t2014 nw290 t2017 0 nch w=1u l=180n
M5368 t2017 t2012 0 0 nch w=1u l=180n
M5369 nw668 t2013 vdd vdd pch w=2u l=180n
M5370 nw668 t2014 vdd vdd pch w=2u l=180n
CT2018 t2018 0 0.1f
M5371 nw668 t2013 t2018 0 nch w=1u l=180n
M5372 t2018 t2014 0 0 nch w=1u l=180n
Cnw668 nw668 0 2f
M5373 nw669 nw650 vdd vdd pch w=2u l=180n
M5374 nw669 nw292 vdd vdd pch w=2u l=180n
CT2019 t2019 0 0.1f
M5375 nw669 nw650 t2019 0 nch w=1u l=180n
M5376 t2019 nw292 0 0 nch w=1u l=180n
Cnw669 nw669 0 2f
M5377 nw670 nw652 0 0 nch w=1u l=180n
M5378 nw670 nw294 0 0 nch w=1u l=180n
CT2020 t2020 0 0.1f
M5379 t2020 nw652 vdd vdd pch w=2u l=180n
M5380 nw670 nw294 t2020 vdd pch w=2u l=180n
Cnw670 nw670 0 2f
CT2021 t2021 0 0.1f
M5381 t2021 nw654 vdd vdd pch w=2u l=180n
M5382 t2021 nw296 vdd vdd pch w=2u l=180n
CT2022 t2022 0 0.1f
M5383 t2021 nw654 t2022 0 nch w=1u l=180n
M5384 t2022 nw296 0 0 nch w=1u l=180n
M5385 nw671 t2021 vdd vdd pch w=2u l=180n
M5386 nw671 t2021 0 0 nch w=1u l=180n
Cnw671 nw671 0 2f
CT2023 t2023 0 0.1f
M5387 t2023 nw656 0 0 nch w=1u l=180n
M5388 t2023 nw298 0 0 nch w=1u l=180n
CT2024 t2024 0 0.1f
M5389 t2024 nw656 vdd vdd pch w=2u l=180n
M5390 t2023 nw298 t2024 vdd pch w=2u l=180n
M5391 nw672 t2023 vdd vdd pch w=2u l=180n
M5392 nw672 t2023 0 0 nch w=1u l=180n
Cnw672 nw672 0 2f
CT2025 t2025 0 0.1f
CT2026 t2026 0 0.1f
CT2027 t2027 0 0.1f
M5393 t2025 nw658 vdd vdd pch w=2u l=180n
M5394 t2025 nw300 vdd vdd pch w=2u l=180n
CT2028 t2028 0 0.1f
M5395 t2025 nw658 t2028 0 nch w=1u l=180n
M5396 t2028 nw300 0 0 nch w=1u l=180n
M5397 t2026 nw658 vdd vdd pch w=2u l=180n
M5398 t2026 t2025 vdd vdd pch w=2u l=180n
CT2029 t2029 0 0.1f
M5399 t2026 nw658 t2029 0 nch w=1u l=180n
M5400 t2029 t2025 0 0 nch w=1u l=180n
M5401 t2027 nw300 vdd vdd pch w=2u l=180n
M5402 t2027 t2025 vdd vdd pch w=2u l=180n
CT2030 t2030 0 0.1f
M5403 t2027 nw300 t2030 0 nch w=1u l=180n
M5404 t2030 t2025 0 0 nch w=1u l=180n
M5405 nw673 t2026 vdd vdd pch w=2u l=180n
M5406 nw673 t2027 vdd vdd pch w=2u l=180n
CT2031 t2031 0 0.1f
M5407 nw673 t2026 t2031 0 nch w=1u l=180n
M5408 t2031 t2027 0 0 nch w=1u l=180n
Cnw673 nw673 0 2f
M5409 nw674 nw660 vdd vdd pch w=2u l=180n
M5410 nw674 nw302 vdd vdd pch w=2u l=180n
CT2032 t2032 0 0.1f
M5411 nw674 nw660 t2032 0 nch w=1u l=180n
M5412 t2032 nw302 0 0 nch w=1u l=180n
Cnw674 nw674 0 2f
M5413 nw675 nw662 0 0 nch w=1u l=180n
M5414 nw675 nw304 0 0 nch w=1u l=180n
CT2033 t2033 0 0.1f
M5415 t2033 nw662 vdd vdd pch w=2u l=180n
M5416 nw675 nw304 t2033 vdd pch w=2u l=180n
Cnw675 nw675 0 2f
CT2034 t2034 0 0.1f
M5417 t2034 nw664 vdd vdd pch w=2u l=180n
M5418 t2034 nw306 vdd vdd pch w=2u l=180n
CT2035 t2035 0 0.1f
M5419 t2034 nw664 t2035 0 nch w=1u l=180n
M5420 t2035 nw306 0 0 nch w=1u l=180n
M5421 nw676 t2034 vdd vdd pch w=2u l=180n
M5422 nw676 t2034 0 0 nch w=1u l=180n
Cnw676 nw676 0 2f
CT2036 t2036 0 0.1f
M5423 t2036 nw666 0 0 nch w=1u l=180n
M5424 t2036 nw308 0 0 nch w=1u l=180n
CT2037 t2037 0 0.1f
M5425 t2037 nw666 vdd vdd pch w=2u l=180n
M5426 t2036 nw308 t2037 vdd pch w=2u l=180n
M5427 nw677 t2036 vdd vdd pch w=2u l=180n
M5428 nw677 t2036 0 0 nch w=1u l=180n
Cnw677 nw677 0 2f
CT2038 t2038 0 0.1f
CT2039 t2039 0 0.1f
CT2040 t2040 0 0.1f
M5429 t2038 nw668 vdd vdd pch w=2u l=180n
M5430 t2038 nw310 vdd vdd pch w=2u l=180n
CT2041 t2041 0 0.1f
M5431 t2038 nw668 t2041 0 nch w=1u l=180n
M5432 t2041 nw310 0 0 nch w=1u l=180n
M5433 t2039 nw668 vdd vdd pch w=2u l=180n
M5434 t2039 t2038 vdd vdd pch w=2u l=180n
CT2042 t2042 0 0.1f
M5435 t2039 nw668 t2042 0 nch w=1u l=180n
M5436 t2042 t2038 0 0 nch w=1u l=180n
M5437 t2040 nw310 vdd vdd pch w=2u l=180n
M5438 t2040 t2038 vdd vdd pch w=2u l=180n
CT2043 t2043 0 0.1f
M5439 t2040 nw310 t2043 0 nch w=1u l=180n
M5440 t2043 t2038 0 0 nch w=1u l=180n
M5441 nw678 t2039 vdd vdd pch w=2u l=180n
M5442 nw678 t2040 vdd vdd pch w=2u l=180n
CT2044 t2044 0 0.1f
M5443 nw678 t2039 t2044 0 nch w=1u l=180n
M5444 t2044 t2040 0 0 nch w=1u l=180n
Cnw678 nw678 0 2f
M5445 nw679 nw670 vdd vdd pch w=2u l=180n
M5446 nw679 nw312 vdd vdd pch w=2u l=180n
CT2045 t2045 0 0.1f
M5447 nw679 nw670 t2045 0 nch w=1u l=180n
M5448 t2045 nw312 0 0 nch w=1u l=180n
Cnw679 nw679 0 2f
M5449 nw680 nw672 0 0 nch w=1u l=180n
M5450 nw680 nw314 0 0 nch w=1u l=180n
CT2046 t2046 0 0.1f
M5451 t2046 nw672 vdd vdd pch w=2u l=180n
M5452 nw680 nw314 t2046 vdd pch w=2u l=180n
Cnw680 nw680 0 2f
CT2047 t2047 0 0.1f
M5453 t2047 nw674 vdd vdd pch w=2u l=180n
M5454 t2047 nw316 vdd vdd pch w=2u l=180n
CT2048 t2048 0 0.1f
M5455 t2047 nw674 t2048 0 nch w=1u l=180n
M5456 t2048 nw316 0 0 nch w=1u l=180n
M5457 nw681 t2047 vdd vdd pch w=2u l=180n
M5458 nw681 t2047 0 0 nch w=1u l=180n
Cnw681 nw681 0 2f
CT2049 t2049 0 0.1f
M5459 t2049 nw676 0 0 nch w=1u l=180n
M5460 t2049 nw318 0 0 nch w=1u l=180n
CT2050 t2050 0 0.1f
M5461 t2050 nw676 vdd vdd pch w=2u l=180n
M5462 t2049 nw318 t2050 vdd pch w=2u l=180n
M5463 nw682 t2049 vdd vdd pch w=2u l=180n
M5464 nw682 t2049 0 0 nch w=1u l=180n
Cnw682 nw682 0 2f
CT2051 t2051 0 0.1f
CT2052 t2052 0 0.1f
CT2053 t2053 0 0.1f
M5465 t2051 nw678 vdd vdd pch w=2u l=180n
M5466 t2051 nw320 vdd vdd pch w=2u l=180n
CT2054 t2054 0 0.1f
M5467 t2051 nw678 t2054 0 nch w=1u l=180n
M5468 t2054 nw320 0 0 nch w=1u l=180n
M5469 t2052 nw678 vdd vdd pch w=2u l=180n
M5470 t2052 t2051 vdd vdd pch w=2u l=180n
CT2055 t2055 0 0.1f
M5471 t2052 nw678 t2055 0 nch w=1u l=180n
M5472 t2055 t2051 0 0 nch w=1u l=180n
M5473 t2053 nw320 vdd vdd pch w=2u l=180n
M5474 t2053 t2051 vdd vdd pch w=2u l=180n
CT2056 t2056 0 0.1f
M5475 t2053 nw320 t2056 0 nch w=1u l=180n
M5476 t2056 t2051 0 0 nch w=1u l=180n
M5477 nw683 t2052 vdd vdd pch w=2u l=180n
M5478 nw683 t2053 vdd vdd pch w=2u l=180n
CT2057 t2057 0 0.1f
M5479 nw683 t2052 t2057 0 nch w=1u l=180n
M5480 t2057 t2053 0 0 nch w=1u l=180n
Cnw683 nw683 0 2f
M5481 nw684 nw680 vdd vdd pch w=2u l=180n
M5482 nw684 nw322 vdd vdd pch w=2u l=180n
CT2058 t2058 0 0.1f
M5483 nw684 nw680 t2058 0 nch w=1u l=180n
M5484 t2058 nw322 0 0 nch w=1u l=180n
Cnw684 nw684 0 2f
M5485 nw685 nw682 0 0 nch w=1u l=180n
M5486 nw685 nw324 0 0 nch w=1u l=180n
CT2059 t2059 0 0.1f
M5487 t2059 nw682 vdd vdd pch w=2u l=180n
M5488 nw685 nw324 t2059 vdd pch w=2u l=180n
Cnw685 nw685 0 2f
CT2060 t2060 0 0.1f
M5489 t2060 nw684 vdd vdd pch w=2u l=180n
M5490 t2060 nw326 vdd vdd pch w=2u l=180n
CT2061 t2061 0 0.1f
M5491 t2060 nw684 t2061 0 nch w=1u l=180n
M5492 t2061 nw326 0 0 nch w=1u l=180n
M5493 nw686 t2060 vdd vdd pch w=2u l=180n
M5494 nw686 t2060 0 0 nch w=1u l=180n
Cnw686 nw686 0 2f
CT2062 t2062 0 0.1f
M5495 t2062 nw686 0 0 nch w=1u l=180n
M5496 t2062 nw328 0 0 nch w=1u l=180n
CT2063 t2063 0 0.1f
M5497 t2063 nw686 vdd vdd pch w=2u l=180n
M5498 t2062 nw328 t2063 vdd pch w=2u l=180n
M5499 nw687 t2062 vdd vdd pch w=2u l=180n
M5500 nw687 t2062 0 0 nch w=1u l=180n
Cnw687 nw687 0 2f
CT2064 t2064 0 0.1f
CT2065 t2065 0 0.1f
CT2066 t2066 0 0.1f
M5501 t2064 nq0 vdd vdd pch w=2u l=180n
M5502 t2064 nw330 vdd vdd pch w=2u l=180n
CT2067 t2067 0 0.1f
M5503 t2064 nq0 t2067 0 nch w=1u l=180n
M5504 t2067 nw330 0 0 nch w=1u l=180n
M5505 t2065 nq0 vdd vdd pch w=2u l=180n
M5506 t2065 t2064 vdd vdd pch w=2u l=180n
CT2068 t2068 0 0.1f
M5507 t2065 nq0 t2068 0 nch w=1u l=180n
M5508 t2068 t2064 0 0 nch w=1u l=180n
M5509 t2066 nw330 vdd vdd pch w=2u l=180n
M5510 t2066 t2064 vdd vdd pch w=2u l=180n
CT2069 t2069 0 0.1f
M5511 t2066 nw330 t2069 0 nch w=1u l=180n
M5512 t2069 t2064 0 0 nch w=1u l=180n
M5513 nw688 t2065 vdd vdd pch w=2u l=180n
M5514 nw688 t2066 vdd vdd pch w=2u l=180n
CT2070 t2070 0 0.1f
M5515 nw688 t2065 t2070 0 nch w=1u l=180n
M5516 t2070 t2066 0 0 nch w=1u l=180n
Cnw688 nw688 0 2f
M5517 nw689 nq1 vdd vdd pch w=2u l=180n
M5518 nw689 nw332 vdd vdd pch w=2u l=180n
CT2071 t2071 0 0.1f
M5519 nw689 nq1 t2071 0 nch w=1u l=180n
M5520 t2071 nw332 0 0 nch w=1u l=180n
Cnw689 nw689 0 2f
M5521 nw690 nq2 0 0 nch w=1u l=180n
M5522 nw690 nw334 0 0 nch w=1u l=180n
CT2072 t2072 0 0.1f
M5523 t2072 nq2 vdd vdd pch w=2u l=180n
M5524 nw690 nw334 t2072 vdd pch w=2u l=180n
Cnw690 nw690 0 2f
CT2073 t2073 0 0.1f
M5525 t2073 nq3 vdd vdd pch w=2u l=180n
M5526 t2073 nw336 vdd vdd pch w=2u l=180n
CT2074 t2074 0 0.1f
M5527 t2073 nq3 t2074 0 nch w=1u l=180n
M5528 t2074 nw336 0 0 nch w=1u l=180n
M5529 nw691 t2073 vdd vdd pch w=2u l=180n
M5530 nw691 t2073 0 0 nch w=1u l=180n
Cnw691 nw691 0 2f
CT2075 t2075 0 0.1f
M5531 t2075 nq4 0 0 nch w=1u l=180n
M5532 t2075 nw338 0 0 nch w=1u l=180n
CT2076 t2076 0 0.1f
M5533 t2076 nq4 vdd vdd pch w=2u l=180n
M5534 t2075 nw338 t2076 vdd pch w=2u l=180n
M5535 nw692 t2075 vdd vdd pch w=2u l=180n
M5536 nw692 t2075 0 0 nch w=1u l=180n
Cnw692 nw692 0 2f
CT2077 t2077 0 0.1f
CT2078 t2078 0 0.1f
CT2079 t2079 0 0.1f
M5537 t2077 nq5 vdd vdd pch w=2u l=180n
M5538 t2077 nw340 vdd vdd pch w=2u l=180n
CT2080 t2080 0 0.1f
M5539 t2077 nq5 t2080 0 nch w=1u l=180n
M5540 t2080 nw340 0 0 nch w=1u l=180n
M5541 t2078 nq5 vdd vdd pch w=2u l=180n
M5542 t2078 t2077 vdd vdd pch w=2u l=180n
CT2081 t2081 0 0.1f
M5543 t2078 nq5 t2081 0 nch w=1u l=180n
M5544 t2081 t2077 0 0 nch w=1u l=180n
M5545 t2079 nw340 vdd vdd pch w=2u l=180n
M5546 t2079 t2077 vdd vdd pch w=2u l=180n
CT2082 t2082 0 0.1f
M5547 t2079 nw340 t2082 0 nch w=1u l=180n
M5548 t2082 t2077 0 0 nch w=1u l=180n
M5549 nw693 t2078 vdd vdd pch w=2u l=180n
M5550 nw693 t2079 vdd vdd pch w=2u l=180n
CT2083 t2083 0 0.1f
M5551 nw693 t2078 t2083 0 nch w=1u l=180n
M5552 t2083 t2079 0 0 nch w=1u l=180n
Cnw693 nw693 0 2f
M5553 nw694 nq6 vdd vdd pch w=2u l=180n
M5554 nw694 nw342 vdd vdd pch w=2u l=180n
CT2084 t2084 0 0.1f
M5555 nw694 nq6 t2084 0 nch w=1u l=180n
M5556 t2084 nw342 0 0 nch w=1u l=180n
Cnw694 nw694 0 2f
M5557 nw695 nq7 0 0 nch w=1u l=180n
M5558 nw695 nw344 0 0 nch w=1u l=180n
CT2085 t2085 0 0.1f
M5559 t2085 nq7 vdd vdd pch w=2u l=180n
M5560 nw695 nw344 t2085 vdd pch w=2u l=180n
Cnw695 nw695 0 2f
CT2086 t2086 0 0.1f
M5561 t2086 nq8 vdd vdd pch w=2u l=180n
M5562 t2086 nw346 vdd vdd pch w=2u l=180n
CT2087 t2087 0 0.1f
M5563 t2086 nq8 t2087 0 nch w=1u l=180n
M5564 t2087 nw346 0 0 nch w=1u l=180n
M5565 nw696 t2086 vdd vdd pch w=2u l=180n
M5566 nw696 t2086 0 0 nch w=1u l=180n
Cnw696 nw696 0 2f
CT2088 t2088 0 0.1f
M5567 t2088 nq9 0 0 nch w=1u l=180n
M5568 t2088 nw348 0 0 nch w=1u l=180n
CT2089 t2089 0 0.1f
M5569 t2089 nq9 vdd vdd pch w=2u l=180n
M5570 t2088 nw348 t2089 vdd pch w=2u l=180n
M5571 nw697 t2088 vdd vdd pch w=2u l=180n
M5572 nw697 t2088 0 0 nch w=1u l=180n
Cnw697 nw697 0 2f
CT2090 t2090 0 0.1f
CT2091 t2091 0 0.1f
CT2092 t2092 0 0.1f
M5573 t2090 nq10 vdd vdd pch w=2u l=180n
M5574 t2090 nw350 vdd vdd pch w=2u l=180n
CT2093 t2093 0 0.1f
M5575 t2090 nq10 t2093 0 nch w=1u l=180n
M5576 t2093 nw350 0 0 nch w=1u l=180n
M5577 t2091 nq10 vdd vdd pch w=2u l=180n
M5578 t2091 t2090 vdd vdd pch w=2u l=180n
CT2094 t2094 0 0.1f
M5579 t2091 nq10 t2094 0 nch w=1u l=180n
M5580 t2094 t2090 0 0 nch w=1u l=180n
M5581 t2092 nw350 vdd vdd pch w=2u l=180n
M5582 t2092 t2090 vdd vdd pch w=2u l=180n
CT2095 t2095 0 0.1f
M5583 t2092 nw350 t2095 0 nch w=1u l=180n
M5584 t2095 t2090 0 0 nch w=1u l=180n
M5585 nw698 t2091 vdd vdd pch w=2u l=180n
M5586 nw698 t2092 vdd vdd pch w=2u l=180n
CT2096 t2096 0 0.1f
M5587 nw698 t2091 t2096 0 nch w=1u l=180n
M5588 t2096 t2092 0 0 nch w=1u l=180n
Cnw698 nw698 0 2f
M5589 nw699 nq11 vdd vdd pch w=2u l=180n
M5590 nw699 nw352 vdd vdd pch w=2u l=180n
CT2097 t2097 0 0.1f
M5591 nw699 nq11 t2097 0 nch w=1u l=180n
M5592 t2097 nw352 0 0 nch w=1u l=180n
Cnw699 nw699 0 2f
M5593 nw700 nq12 0 0 nch w=1u l=180n
M5594 nw700 nw354 0 0 nch w=1u l=180n
CT2098 t2098 0 0.1f
M5595 t2098 nq12 vdd vdd pch w=2u l=180n
M5596 nw700 nw354 t2098 vdd pch w=2u l=180n
Cnw700 nw700 0 2f
CT2099 t2099 0 0.1f
M5597 t2099 nq13 vdd vdd pch w=2u l=180n
M5598 t2099 nw356 vdd vdd pch w=2u l=180n
CT2100 t2100 0 0.1f
M5599 t2099 nq13 t2100 0 nch w=1u l=180n
M5600 t2100 nw356 0 0 nch w=1u l=180n
M5601 nw701 t2099 vdd vdd pch w=2u l=180n
M5602 nw701 t2099 0 0 nch w=1u l=180n
Cnw701 nw701 0 2f
CT2101 t2101 0 0.1f
M5603 t2101 nq14 0 0 nch w=1u l=180n
M5604 t2101 nw358 0 0 nch w=1u l=180n
CT2102 t2102 0 0.1f
M5605 t2102 nq14 vdd vdd pch w=2u l=180n
M5606 t2101 nw358 t2102 vdd pch w=2u l=180n
M5607 nw702 t2101 vdd vdd pch w=2u l=180n
M5608 nw702 t2101 0 0 nch w=1u l=180n
Cnw702 nw702 0 2f
CT2103 t2103 0 0.1f
CT2104 t2104 0 0.1f
CT2105 t2105 0 0.1f
M5609 t2103 nq15 vdd vdd pch w=2u l=180n
M5610 t2103 nw360 vdd vdd pch w=2u l=180n
CT2106 t2106 0 0.1f
M5611 t2103 nq15 t2106 0 nch w=1u l=180n
M5612 t2106 nw360 0 0 nch w=1u l=180n
M5613 t2104 nq15 vdd vdd pch w=2u l=180n
M5614 t2104 t2103 vdd vdd pch w=2u l=180n
CT2107 t2107 0 0.1f
M5615 t2104 nq15 t2107 0 nch w=1u l=180n
M5616 t2107 t2103 0 0 nch w=1u l=180n
M5617 t2105 nw360 vdd vdd pch w=2u l=180n
M5618 t2105 t2103 vdd vdd pch w=2u l=180n
CT2108 t2108 0 0.1f
M5619 t2105 nw360 t2108 0 nch w=1u l=180n
M5620 t2108 t2103 0 0 nch w=1u l=180n
M5621 nw703 t2104 vdd vdd pch w=2u l=180n
M5622 nw703 t2105 vdd vdd pch w=2u l=180n
CT2109 t2109 0 0.1f
M5623 nw703 t2104 t2109 0 nch w=1u l=180n
M5624 t2109 t2105 0 0 nch w=1u l=180n
Cnw703 nw703 0 2f
M5625 nw704 nq16 vdd vdd pch w=2u l=180n
M5626 nw704 nw362 vdd vdd pch w=2u l=180n
CT2110 t2110 0 0.1f
M5627 nw704 nq16 t2110 0 nch w=1u l=180n
M5628 t2110 nw362 0 0 nch w=1u l=180n
Cnw704 nw704 0 2f
M5629 nw705 nq17 0 0 nch w=1u l=180n
M5630 nw705 nw364 0 0 nch w=1u l=180n
CT2111 t2111 0 0.1f
M5631 t2111 nq17 vdd vdd pch w=2u l=180n
M5632 nw705 nw364 t2111 vdd pch w=2u l=180n
Cnw705 nw705 0 2f
CT2112 t2112 0 0.1f
M5633 t2112 nq18 vdd vdd pch w=2u l=180n
M5634 t2112 nw366 vdd vdd pch w=2u l=180n
CT2113 t2113 0 0.1f
M5635 t2112 nq18 t2113 0 nch w=1u l=180n
M5636 t2113 nw366 0 0 nch w=1u l=180n
M5637 nw706 t2112 vdd vdd pch w=2u l=180n
M5638 nw706 t2112 0 0 nch w=1u l=180n
Cnw706 nw706 0 2f
CT2114 t2114 0 0.1f
M5639 t2114 nq19 0 0 nch w=1u l=180n
M5640 t2114 nw368 0 0 nch w=1u l=180n
CT2115 t2115 0 0.1f
M5641 t2115 nq19 vdd vdd pch w=2u l=180n
M5642 t2114 nw368 t2115 vdd pch w=2u l=180n
M5643 nw707 t2114 vdd vdd pch w=2u l=180n
M5644 nw707 t2114 0 0 nch w=1u l=180n
Cnw707 nw707 0 2f
CT2116 t2116 0 0.1f
CT2117 t2117 0 0.1f
CT2118 t2118 0 0.1f
M5645 t2116 nq20 vdd vdd pch w=2u l=180n
M5646 t2116 nw370 vdd vdd pch w=2u l=180n
CT2119 t2119 0 0.1f
M5647 t2116 nq20 t2119 0 nch w=1u l=180n
M5648 t2119 nw370 0 0 nch w=1u l=180n
M5649 t2117 nq20 vdd vdd pch w=2u l=180n
M5650 t2117 t2116 vdd vdd pch w=2u l=180n
CT2120 t2120 0 0.1f
M5651 t2117 nq20 t2120 0 nch w=1u l=180n
M5652 t2120 t2116 0 0 nch w=1u l=180n
M5653 t2118 nw370 vdd vdd pch w=2u l=180n
M5654 t2118 t2116 vdd vdd pch w=2u l=180n
CT2121 t2121 0 0.1f
M5655 t2118 nw370 t2121 0 nch w=1u l=180n
M5656 t2121 t2116 0 0 nch w=1u l=180n
M5657 nw708 t2117 vdd vdd pch w=2u l=180n
M5658 nw708 t2118 vdd vdd pch w=2u l=180n
CT2122 t2122 0 0.1f
M5659 nw708 t2117 t2122 0 nch w=1u l=180n
M5660 t2122 t2118 0 0 nch w=1u l=180n
Cnw708 nw708 0 2f
M5661 nw709 nq21 vdd vdd pch w=2u l=180n
M5662 nw709 nw372 vdd vdd pch w=2u l=180n
CT2123 t2123 0 0.1f
M5663 nw709 nq21 t2123 0 nch w=1u l=180n
M5664 t2123 nw372 0 0 nch w=1u l=180n
Cnw709 nw709 0 2f
M5665 nw710 nq22 0 0 nch w=1u l=180n
M5666 nw710 nw374 0 0 nch w=1u l=180n
CT2124 t2124 0 0.1f
M5667 t2124 nq22 vdd vdd pch w=2u l=180n
M5668 nw710 nw374 t2124 vdd pch w=2u l=180n
Cnw710 nw710 0 2f
CT2125 t2125 0 0.1f
M5669 t2125 nq23 vdd vdd pch w=2u l=180n
M5670 t2125 nw376 vdd vdd pch w=2u l=180n
CT2126 t2126 0 0.1f
M5671 t2125 nq23 t2126 0 nch w=1u l=180n
M5672 t2126 nw376 0 0 nch w=1u l=180n
M5673 nw711 t2125 vdd vdd pch w=2u l=180n
M5674 nw711 t2125 0 0 nch w=1u l=180n
Cnw711 nw711 0 2f
CT2127 t2127 0 0.1f
M5675 t2127 nq24 0 0 nch w=1u l=180n
M5676 t2127 nw378 0 0 nch w=1u l=180n
CT2128 t2128 0 0.1f
M5677 t2128 nq24 vdd vdd pch w=2u l=180n
M5678 t2127 nw378 t2128 vdd pch w=2u l=180n
M5679 nw712 t2127 vdd vdd pch w=2u l=180n
M5680 nw712 t2127 0 0 nch w=1u l=180n
Cnw712 nw712 0 2f
CT2129 t2129 0 0.1f
CT2130 t2130 0 0.1f
CT2131 t2131 0 0.1f
M5681 t2129 nq25 vdd vdd pch w=2u l=180n
M5682 t2129 nw380 vdd vdd pch w=2u l=180n
CT2132 t2132 0 0.1f
M5683 t2129 nq25 t2132 0 nch w=1u l=180n
M5684 t2132 nw380 0 0 nch w=1u l=180n
M5685 t2130 nq25 vdd vdd pch w=2u l=180n
M5686 t2130 t2129 vdd vdd pch w=2u l=180n
CT2133 t2133 0 0.1f
M5687 t2130 nq25 t2133 0 nch w=1u l=180n
M5688 t2133 t2129 0 0 nch w=1u l=180n
M5689 t2131 nw380 vdd vdd pch w=2u l=180n
M5690 t2131 t2129 vdd vdd pch w=2u l=180n
CT2134 t2134 0 0.1f
M5691 t2131 nw380 t2134 0 nch w=1u l=180n
M5692 t2134 t2129 0 0 nch w=1u l=180n
M5693 nw713 t2130 vdd vdd pch w=2u l=180n
M5694 nw713 t2131 vdd vdd pch w=2u l=180n
CT2135 t2135 0 0.1f
M5695 nw713 t2130 t2135 0 nch w=1u l=180n
M5696 t2135 t2131 0 0 nch w=1u l=180n
Cnw713 nw713 0 2f
M5697 nw714 nq26 vdd vdd pch w=2u l=180n
M5698 nw714 nw382 vdd vdd pch w=2u l=180n
CT2136 t2136 0 0.1f
M5699 nw714 nq26 t2136 0 nch w=1u l=180n
M5700 t2136 nw382 0 0 nch w=1u l=180n
Cnw714 nw714 0 2f
M5701 nw715 nq27 0 0 nch w=1u l=180n
M5702 nw715 nw384 0 0 nch w=1u l=180n
CT2137 t2137 0 0.1f
M5703 t2137 nq27 vdd vdd pch w=2u l=180n
M5704 nw715 nw384 t2137 vdd pch w=2u l=180n
Cnw715 nw715 0 2f
CT2138 t2138 0 0.1f
M5705 t2138 nq28 vdd vdd pch w=2u l=180n
M5706 t2138 nw386 vdd vdd pch w=2u l=180n
CT2139 t2139 0 0.1f
M5707 t2138 nq28 t2139 0 nch w=1u l=180n
M5708 t2139 nw386 0 0 nch w=1u l=180n
M5709 nw716 t2138 vdd vdd pch w=2u l=180n
M5710 nw716 t2138 0 0 nch w=1u l=180n
Cnw716 nw716 0 2f
CT2140 t2140 0 0.1f
M5711 t2140 nq29 0 0 nch w=1u l=180n
M5712 t2140 nw388 0 0 nch w=1u l=180n
CT2141 t2141 0 0.1f
M5713 t2141 nq29 vdd vdd pch w=2u l=180n
M5714 t2140 nw388 t2141 vdd pch w=2u l=180n
M5715 nw717 t2140 vdd vdd pch w=2u l=180n
M5716 nw717 t2140 0 0 nch w=1u l=180n
Cnw717 nw717 0 2f
CT2142 t2142 0 0.1f
CT2143 t2143 0 0.1f
CT2144 t2144 0 0.1f
M5717 t2142 nq30 vdd vdd pch w=2u l=180n
M5718 t2142 nw390 vdd vdd pch w=2u l=180n
CT2145 t2145 0 0.1f
M5719 t2142 nq30 t2145 0 nch w=1u l=180n
M5720 t2145 nw390 0 0 nch w=1u l=180n
M5721 t2143 nq30 vdd vdd pch w=2u l=180n
M5722 t2143 t2142 vdd vdd pch w=2u l=180n
CT2146 t2146 0 0.1f
M5723 t2143 nq30 t2146 0 nch w=1u l=180n
M5724 t2146 t2142 0 0 nch w=1u l=180n
M5725 t2144 nw390 vdd vdd pch w=2u l=180n
M5726 t2144 t2142 vdd vdd pch w=2u l=180n
CT2147 t2147 0 0.1f
M5727 t2144 nw390 t2147 0 nch w=1u l=180n
M5728 t2147 t2142 0 0 nch w=1u l=180n
M5729 nw718 t2143 vdd vdd pch w=2u l=180n
M5730 nw718 t2144 vdd vdd pch w=2u l=180n
CT2148 t2148 0 0.1f
M5731 nw718 t2143 t2148 0 nch w=1u l=180n
M5732 t2148 t2144 0 0 nch w=1u l=180n
Cnw718 nw718 0 2f
M5733 nw719 nq31 vdd vdd pch w=2u l=180n
M5734 nw719 nw392 vdd vdd pch w=2u l=180n
CT2149 t2149 0 0.1f
M5735 nw719 nq31 t2149 0 nch w=1u l=180n
M5736 t2149 nw392 0 0 nch w=1u l=180n
Cnw719 nw719 0 2f
M5737 nw720 nq32 0 0 nch w=1u l=180n
M5738 nw720 nw394 0 0 nch w=1u l=180n
CT2150 t2150 0 0.1f
M5739 t2150 nq32 vdd vdd pch w=2u l=180n
M5740 nw720 nw394 t2150 vdd pch w=2u l=180n
Cnw720 nw720 0 2f
CT2151 t2151 0 0.1f
M5741 t2151 nq33 vdd vdd pch w=2u l=180n
M5742 t2151 nw396 vdd vdd pch w=2u l=180n
CT2152 t2152 0 0.1f
M5743 t2151 nq33 t2152 0 nch w=1u l=180n
M5744 t2152 nw396 0 0 nch w=1u l=180n
M5745 nw721 t2151 vdd vdd pch w=2u l=180n
M5746 nw721 t2151 0 0 nch w=1u l=180n
Cnw721 nw721 0 2f
CT2153 t2153 0 0.1f
M5747 t2153 nq34 0 0 nch w=1u l=180n
M5748 t2153 nw398 0 0 nch w=1u l=180n
CT2154 t2154 0 0.1f
M5749 t2154 nq34 vdd vdd pch w=2u l=180n
M5750 t2153 nw398 t2154 vdd pch w=2u l=180n
M5751 nw722 t2153 vdd vdd pch w=2u l=180n
M5752 nw722 t2153 0 0 nch w=1u l=180n
Cnw722 nw722 0 2f
CT2155 t2155 0 0.1f
CT2156 t2156 0 0.1f
CT2157 t2157 0 0.1f
M5753 t2155 nq35 vdd vdd pch w=2u l=180n
M5754 t2155 nw400 vdd vdd pch w=2u l=180n
CT2158 t2158 0 0.1f
M5755 t2155 nq35 t2158 0 nch w=1u l=180n
M5756 t2158 nw400 0 0 nch w=1u l=180n
M5757 t2156 nq35 vdd vdd pch w=2u l=180n
M5758 t2156 t2155 vdd vdd pch w=2u l=180n
CT2159 t2159 0 0.1f
M5759 t2156 nq35 t2159 0 nch w=1u l=180n
M5760 t2159 t2155 0 0 nch w=1u l=180n
M5761 t2157 nw400 vdd vdd pch w=2u l=180n
M5762 t2157 t2155 vdd vdd pch w=2u l=180n
CT2160 t2160 0 0.1f
M5763 t2157 nw400 t2160 0 nch w=1u l=180n
M5764 t2160 t2155 0 0 nch w=1u l=180n
M5765 nw723 t2156 vdd vdd pch w=2u l=180n
M5766 nw723 t2157 vdd vdd pch w=2u l=180n
CT2161 t2161 0 0.1f
M5767 nw723 t2156 t2161 0 nch w=1u l=180n
M5768 t2161 t2157 0 0 nch w=1u l=180n
Cnw723 nw723 0 2f
M5769 nw724 nq36 vdd vdd pch w=2u l=180n
M5770 nw724 nw402 vdd vdd pch w=2u l=180n
CT2162 t2162 0 0.1f
M5771 nw724 nq36 t2162 0 nch w=1u l=180n
M5772 t2162 nw402 0 0 nch w=1u l=180n
Cnw724 nw724 0 2f
M5773 nw725 nq37 0 0 nch w=1u l=180n
M5774 nw725 nw404 0 0 nch w=1u l=180n
CT2163 t2163 0 0.1f
M5775 t2163 nq37 vdd vdd pch w=2u l=180n
M5776 nw725 nw404 t2163 vdd pch w=2u l=180n
Cnw725 nw725 0 2f
CT2164 t2164 0 0.1f
M5777 t2164 nq38 vdd vdd pch w=2u l=180n
M5778 t2164 nw406 vdd vdd pch w=2u l=180n
CT2165 t2165 0 0.1f
M5779 t2164 nq38 t2165 0 nch w=1u l=180n
M5780 t2165 nw406 0 0 nch w=1u l=180n
M5781 nw726 t2164 vdd vdd pch w=2u l=180n
M5782 nw726 t2164 0 0 nch w=1u l=180n
Cnw726 nw726 0 2f
CT2166 t2166 0 0.1f
M5783 t2166 nq39 0 0 nch w=1u l=180n
M5784 t2166 nw408 0 0 nch w=1u l=180n
CT2167 t2167 0 0.1f
M5785 t2167 nq39 vdd vdd pch w=2u l=180n
M5786 t2166 nw408 t2167 vdd pch w=2u l=180n
M5787 nw727 t2166 vdd vdd pch w=2u l=180n
M5788 nw727 t2166 0 0 nch w=1u l=180n
Cnw727 nw727 0 2f
CT2168 t2168 0 0.1f
CT2169 t2169 0 0.1f
CT2170 t2170 0 0.1f
M5789 t2168 nq40 vdd vdd pch w=2u l=180n
M5790 t2168 nw410 vdd vdd pch w=2u l=180n
CT2171 t2171 0 0.1f
M5791 t2168 nq40 t2171 0 nch w=1u l=180n
M5792 t2171 nw410 0 0 nch w=1u l=180n
M5793 t2169 nq40 vdd vdd pch w=2u l=180n
M5794 t2169 t2168 vdd vdd pch w=2u l=180n
CT2172 t2172 0 0.1f
M5795 t2169 nq40 t2172 0 nch w=1u l=180n
M5796 t2172 t2168 0 0 nch w=1u l=180n
M5797 t2170 nw410 vdd vdd pch w=2u l=180n
M5798 t2170 t2168 vdd vdd pch w=2u l=180n
CT2173 t2173 0 0.1f
M5799 t2170 nw410 t2173 0 nch w=1u l=180n
M5800 t2173 t2168 0 0 nch w=1u l=180n
M5801 nw728 t2169 vdd vdd pch w=2u l=180n
M5802 nw728 t2170 vdd vdd pch w=2u l=180n
CT2174 t2174 0 0.1f
M5803 nw728 t2169 t2174 0 nch w=1u l=180n
M5804 t2174 t2170 0 0 nch w=1u l=180n
Cnw728 nw728 0 2f
M5805 nw729 nq41 vdd vdd pch w=2u l=180n
M5806 nw729 nw412 vdd vdd pch w=2u l=180n
CT2175 t2175 0 0.1f
M5807 nw729 nq41 t2175 0 nch w=1u l=180n
M5808 t2175 nw412 0 0 nch w=1u l=180n
Cnw729 nw729 0 2f
M5809 nw730 nq42 0 0 nch w=1u l=180n
M5810 nw730 nw414 0 0 nch w=1u l=180n
CT2176 t2176 0 0.1f
M5811 t2176 nq42 vdd vdd pch w=2u l=180n
M5812 nw730 nw414 t2176 vdd pch w=2u l=180n
Cnw730 nw730 0 2f
CT2177 t2177 0 0.1f
M5813 t2177 nq43 vdd vdd pch w=2u l=180n
M5814 t2177 nw416 vdd vdd pch w=2u l=180n
CT2178 t2178 0 0.1f
M5815 t2177 nq43 t2178 0 nch w=1u l=180n
M5816 t2178 nw416 0 0 nch w=1u l=180n
M5817 nw731 t2177 vdd vdd pch w=2u l=180n
M5818 nw731 t2177 0 0 nch w=1u l=180n
Cnw731 nw731 0 2f
CT2179 t2179 0 0.1f
M5819 t2179 nq44 0 0 nch w=1u l=180n
M5820 t2179 nw418 0 0 nch w=1u l=180n
CT2180 t2180 0 0.1f
M5821 t2180 nq44 vdd vdd pch w=2u l=180n
M5822 t2179 nw418 t2180 vdd pch w=2u l=180n
M5823 nw732 t2179 vdd vdd pch w=2u l=180n
M5824 nw732 t2179 0 0 nch w=1u l=180n
Cnw732 nw732 0 2f
CT2181 t2181 0 0.1f
CT2182 t2182 0 0.1f
CT2183 t2183 0 0.1f
M5825 t2181 nq45 vdd vdd pch w=2u l=180n
M5826 t2181 nw420 vdd vdd pch w=2u l=180n
CT2184 t2184 0 0.1f
M5827 t2181 nq45 t2184 0 nch w=1u l=180n
M5828 t2184 nw420 0 0 nch w=1u l=180n
M5829 t2182 nq45 vdd vdd pch w=2u l=180n
M5830 t2182 t2181 vdd vdd pch w=2u l=180n
CT2185 t2185 0 0.1f
M5831 t2182 nq45 t2185 0 nch w=1u l=180n
M5832 t2185 t2181 0 0 nch w=1u l=180n
M5833 t2183 nw420 vdd vdd pch w=2u l=180n
M5834 t2183 t2181 vdd vdd pch w=2u l=180n
CT2186 t2186 0 0.1f
M5835 t2183 nw420 t2186 0 nch w=1u l=180n
M5836 t2186 t2181 0 0 nch w=1u l=180n
M5837 nw733 t2182 vdd vdd pch w=2u l=180n
M5838 nw733 t2183 vdd vdd pch w=2u l=180n
CT2187 t2187 0 0.1f
M5839 nw733 t2182 t2187 0 nch w=1u l=180n
M5840 t2187 t2183 0 0 nch w=1u l=180n
Cnw733 nw733 0 2f
M5841 nw734 nq46 vdd vdd pch w=2u l=180n
M5842 nw734 nw422 vdd vdd pch w=2u l=180n
CT2188 t2188 0 0.1f
M5843 nw734 nq46 t2188 0 nch w=1u l=180n
M5844 t2188 nw422 0 0 nch w=1u l=180n
Cnw734 nw734 0 2f
M5845 nw735 nq47 0 0 nch w=1u l=180n
M5846 nw735 nw424 0 0 nch w=1u l=180n
CT2189 t2189 0 0.1f
M5847 t2189 nq47 vdd vdd pch w=2u l=180n
M5848 nw735 nw424 t2189 vdd pch w=2u l=180n
Cnw735 nw735 0 2f
CT2190 t2190 0 0.1f
M5849 t2190 nq48 vdd vdd pch w=2u l=180n
M5850 t2190 nw426 vdd vdd pch w=2u l=180n
CT2191 t2191 0 0.1f
M5851 t2190 nq48 t2191 0 nch w=1u l=180n
M5852 t2191 nw426 0 0 nch w=1u l=180n
M5853 nw736 t2190 vdd vdd pch w=2u l=180n
M5854 nw736 t2190 0 0 nch w=1u l=180n
Cnw736 nw736 0 2f
CT2192 t2192 0 0.1f
M5855 t2192 nq49 0 0 nch w=1u l=180n
M5856 t2192 nw428 0 0 nch w=1u l=180n
CT2193 t2193 0 0.1f
M5857 t2193 nq49 vdd vdd pch w=2u l=180n
M5858 t2192 nw428 t2193 vdd pch w=2u l=180n
M5859 nw737 t2192 vdd vdd pch w=2u l=180n
M5860 nw737 t2192 0 0 nch w=1u l=180n
Cnw737 nw737 0 2f
CT2194 t2194 0 0.1f
CT2195 t2195 0 0.1f
CT2196 t2196 0 0.1f
M5861 t2194 nq50 vdd vdd pch w=2u l=180n
M5862 t2194 nw430 vdd vdd pch w=2u l=180n
CT2197 t2197 0 0.1f
M5863 t2194 nq50 t2197 0 nch w=1u l=180n
M5864 t2197 nw430 0 0 nch w=1u l=180n
M5865 t2195 nq50 vdd vdd pch w=2u l=180n
M5866 t2195 t2194 vdd vdd pch w=2u l=180n
CT2198 t2198 0 0.1f
M5867 t2195 nq50 t2198 0 nch w=1u l=180n
M5868 t2198 t2194 0 0 nch w=1u l=180n
M5869 t2196 nw430 vdd vdd pch w=2u l=180n
M5870 t2196 t2194 vdd vdd pch w=2u l=180n
CT2199 t2199 0 0.1f
M5871 t2196 nw430 t2199 0 nch w=1u l=180n
M5872 t2199 t2194 0 0 nch w=1u l=180n
M5873 nw738 t2195 vdd vdd pch w=2u l=180n
M5874 nw738 t2196 vdd vdd pch w=2u l=180n
CT2200 t2200 0 0.1f
M5875 nw738 t2195 t2200 0 nch w=1u l=180n
M5876 t2200 t2196 0 0 nch w=1u l=180n
Cnw738 nw738 0 2f
M5877 nw739 nq51 vdd vdd pch w=2u l=180n
M5878 nw739 nw432 vdd vdd pch w=2u l=180n
CT2201 t2201 0 0.1f
M5879 nw739 nq51 t2201 0 nch w=1u l=180n
M5880 t2201 nw432 0 0 nch w=1u l=180n
Cnw739 nw739 0 2f
M5881 nw740 nq52 0 0 nch w=1u l=180n
M5882 nw740 nw434 0 0 nch w=1u l=180n
CT2202 t2202 0 0.1f
M5883 t2202 nq52 vdd vdd pch w=2u l=180n
M5884 nw740 nw434 t2202 vdd pch w=2u l=180n
Cnw740 nw740 0 2f
CT2203 t2203 0 0.1f
M5885 t2203 nq53 vdd vdd pch w=2u l=180n
M5886 t2203 nw436 vdd vdd pch w=2u l=180n
CT2204 t2204 0 0.1f
M5887 t2203 nq53 t2204 0 nch w=1u l=180n
M5888 t2204 nw436 0 0 nch w=1u l=180n
M5889 nw741 t2203 vdd vdd pch w=2u l=180n
M5890 nw741 t2203 0 0 nch w=1u l=180n
Cnw741 nw741 0 2f
CT2205 t2205 0 0.1f
M5891 t2205 nq54 0 0 nch w=1u l=180n
M5892 t2205 nw438 0 0 nch w=1u l=180n
CT2206 t2206 0 0.1f
M5893 t2206 nq54 vdd vdd pch w=2u l=180n
M5894 t2205 nw438 t2206 vdd pch w=2u l=180n
M5895 nw742 t2205 vdd vdd pch w=2u l=180n
M5896 nw742 t2205 0 0 nch w=1u l=180n
Cnw742 nw742 0 2f
CT2207 t2207 0 0.1f
CT2208 t2208 0 0.1f
CT2209 t2209 0 0.1f
M5897 t2207 nq55 vdd vdd pch w=2u l=180n
M5898 t2207 nw440 vdd vdd pch w=2u l=180n
CT2210 t2210 0 0.1f
M5899 t2207 nq55 t2210 0 nch w=1u l=180n
M5900 t2210 nw440 0 0 nch w=1u l=180n
M5901 t2208 nq55 vdd vdd pch w=2u l=180n
M5902 t2208 t2207 vdd vdd pch w=2u l=180n
CT2211 t2211 0 0.1f
M5903 t2208 nq55 t2211 0 nch w=1u l=180n
M5904 t2211 t2207 0 0 nch w=1u l=180n
M5905 t2209 nw440 vdd vdd pch w=2u l=180n
M5906 t2209 t2207 vdd vdd pch w=2u l=180n
CT2212 t2212 0 0.1f
M5907 t2209 nw440 t2212 0 nch w=1u l=180n
M5908 t2212 t2207 0 0 nch w=1u l=180n
M5909 nw743 t2208 vdd vdd pch w=2u l=180n
M5910 nw743 t2209 vdd vdd pch w=2u l=180n
CT2213 t2213 0 0.1f
M5911 nw743 t2208 t2213 0 nch w=1u l=180n
M5912 t2213 t2209 0 0 nch w=1u l=180n
Cnw743 nw743 0 2f
M5913 nw744 nq56 vdd vdd pch w=2u l=180n
M5914 nw744 nw442 vdd vdd pch w=2u l=180n
CT2214 t2214 0 0.1f
M5915 nw744 nq56 t2214 0 nch w=1u l=180n
M5916 t2214 nw442 0 0 nch w=1u l=180n
Cnw744 nw744 0 2f
M5917 nw745 nq57 0 0 nch w=1u l=180n
M5918 nw745 nw444 0 0 nch w=1u l=180n
CT2215 t2215 0 0.1f
M5919 t2215 nq57 vdd vdd pch w=2u l=180n
M5920 nw745 nw444 t2215 vdd pch w=2u l=180n
Cnw745 nw745 0 2f
CT2216 t2216 0 0.1f
M5921 t2216 nq58 vdd vdd pch w=2u l=180n
M5922 t2216 nw446 vdd vdd pch w=2u l=180n
CT2217 t2217 0 0.1f
M5923 t2216 nq58 t2217 0 nch w=1u l=180n
M5924 t2217 nw446 0 0 nch w=1u l=180n
M5925 nw746 t2216 vdd vdd pch w=2u l=180n
M5926 nw746 t2216 0 0 nch w=1u l=180n
Cnw746 nw746 0 2f
CT2218 t2218 0 0.1f
M5927 t2218 nq59 0 0 nch w=1u l=180n
M5928 t2218 nw448 0 0 nch w=1u l=180n
CT2219 t2219 0 0.1f
M5929 t2219 nq59 vdd vdd pch w=2u l=180n
M5930 t2218 nw448 t2219 vdd pch w=2u l=180n
M5931 nw747 t2218 vdd vdd pch w=2u l=180n
M5932 nw747 t2218 0 0 nch w=1u l=180n
Cnw747 nw747 0 2f
CT2220 t2220 0 0.1f
CT2221 t2221 0 0.1f
CT2222 t2222 0 0.1f
M5933 t2220 nq60 vdd vdd pch w=2u l=180n
M5934 t2220 nw450 vdd vdd pch w=2u l=180n
CT2223 t2223 0 0.1f
M5935 t2220 nq60 t2223 0 nch w=1u l=180n
M5936 t2223 nw450 0 0 nch w=1u l=180n
M5937 t2221 nq60 vdd vdd pch w=2u l=180n
M5938 t2221 t2220 vdd vdd pch w=2u l=180n
CT2224 t2224 0 0.1f
M5939 t2221 nq60 t2224 0 nch w=1u l=180n
M5940 t2224 t2220 0 0 nch w=1u l=180n
M5941 t2222 nw450 vdd vdd pch w=2u l=180n
M5942 t2222 t2220 vdd vdd pch w=2u l=180n
CT2225 t2225 0 0.1f
M5943 t2222 nw450 t2225 0 nch w=1u l=180n
M5944 t2225 t2220 0 0 nch w=1u l=180n
M5945 nw748 t2221 vdd vdd pch w=2u l=180n
M5946 nw748 t2222 vdd vdd pch w=2u l=180n
CT2226 t2226 0 0.1f
M5947 nw748 t2221 t2226 0 nch w=1u l=180n
M5948 t2226 t2222 0 0 nch w=1u l=180n
Cnw748 nw748 0 2f
CT2227 t2227 0 0.1f
M5949 t2227 nw748 vdd vdd pch w=2u l=180n
M5950 t2227 nw748 0 0 nch w=1u l=180n
M5951 no0 t2227 vdd vdd pch w=2u l=180n
M5952 no0 t2227 0 0 nch w=1u l=180n
Cno0 no0 0 2f
CT2228 t2228 0 0.1f
M5953 t2228 nw747 vdd vdd pch w=2u l=180n
M5954 t2228 nw747 0 0 nch w=1u l=180n
M5955 no1 t2228 vdd vdd pch w=2u l=180n
M5956 no1 t2228 0 0 nch w=1u l=180n
Cno1 no1 0 2f
CT2229 t2229 0 0.1f
M5957 t2229 nw746 vdd vdd pch w=2u l=180n
M5958 t2229 nw746 0 0 nch w=1u l=180n
M5959 no2 t2229 vdd vdd pch w=2u l=180n
M5960 no2 t2229 0 0 nch w=1u l=180n
Cno2 no2 0 2f
CT2230 t2230 0 0.1f
M5961 t2230 nw745 vdd vdd pch w=2u l=180n
M5962 t2230 nw745 0 0 nch w=1u l=180n
M5963 no3 t2230 vdd vdd pch w=2u l=180n
M5964 no3 t2230 0 0 nch w=1u l=180n
Cno3 no3 0 2f
CT2231 t2231 0 0.1f
M5965 t2231 nw744 vdd vdd pch w=2u l=180n
M5966 t2231 nw744 0 0 nch w=1u l=180n
M5967 no4 t2231 vdd vdd pch w=2u l=180n
M5968 no4 t2231 0 0 nch w=1u l=180n
Cno4 no4 0 2f
CT2232 t2232 0 0.1f
M5969 t2232 nw743 vdd vdd pch w=2u l=180n
M5970 t2232 nw743 0 0 nch w=1u l=180n
M5971 no5 t2232 vdd vdd pch w=2u l=180n
M5972 no5 t2232 0 0 nch w=1u l=180n
Cno5 no5 0 2f
CT2233 t2233 0 0.1f
M5973 t2233 nw742 vdd vdd pch w=2u l=180n
M5974 t2233 nw742 0 0 nch w=1u l=180n
M5975 no6 t2233 vdd vdd pch w=2u l=180n
M5976 no6 t2233 0 0 nch w=1u l=180n
Cno6 no6 0 2f
CT2234 t2234 0 0.1f
M5977 t2234 nw741 vdd vdd pch w=2u l=180n
M5978 t2234 nw741 0 0 nch w=1u l=180n
M5979 no7 t2234 vdd vdd pch w=2u l=180n
M5980 no7 t2234 0 0 nch w=1u l=180n
Cno7 no7 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: nw1 nw3 nw5 nw7 nw9 nw11 nw13 nw15 nw17 nw19 nw21 nw23 nw25 nw27 nw29 nw31 nw33 nw35 nw37 nw39 nw41 nw43 nw45 nw47 nw49 nw51 nw53 nw55 nw57 nw59 nw61 nw63 nw65 nw67 nw69 nw71 nw73 nw75 nw77 nw79 nw81 nw83 nw85 nw87 nw89 nw91 nw93 nw95 nw97 nw99 nw101 nw103 nw105 nw107 nw109 nw111 nw113 nw115 nw117 nw119 nw121 nw123 nw125 nw127 nw129 nw131 nw133 nw135 nw137 nw139 nw141 nw143 nw145 nw147 no0 no1 no2 no3 no4 no5 no6 no7
.end
