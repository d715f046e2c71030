* c432 (c432: 27-channel interrupt controller (priority encoder)): 131 gates, 740 transistors
VDD vdd 0 DC 1.8
VIN0 nreq0 0 PULSE(0 1.8 5e-10 20p 20p 1e-09 2e-09)
VIN1 nreq1 0 PULSE(0 1.8 1e-09 20p 20p 2e-09 4e-09)
VIN2 nreq2 0 PULSE(0 1.8 2e-09 20p 20p 4e-09 8e-09)
VIN3 nreq3 0 PULSE(0 1.8 4e-09 20p 20p 8e-09 1.6e-08)
VIN4 nreq4 0 PULSE(0 1.8 8e-09 20p 20p 1.6e-08 3.2e-08)
VIN5 nreq5 0 PULSE(0 1.8 1.6e-08 20p 20p 3.2e-08 6.4e-08)
VIN6 nreq6 0 PULSE(0 1.8 3.2e-08 20p 20p 6.4e-08 1.28e-07)
VIN7 nreq7 0 PULSE(0 1.8 6.4e-08 20p 20p 1.28e-07 2.56e-07)
VIN8 nreq8 0 PULSE(0 1.8 1.28e-07 20p 20p 2.56e-07 5.12e-07)
VIN9 nreq9 0 PULSE(0 1.8 2.56e-07 20p 20p 5.12e-07 1.024e-06)
VIN10 nreq10 0 PULSE(0 1.8 5.12e-07 20p 20p 1.024e-06 2.048e-06)
VIN11 nreq11 0 PULSE(0 1.8 1.024e-06 20p 20p 2.048e-06 4.096e-06)
VIN12 nreq12 0 PULSE(0 1.8 2.048e-06 20p 20p 4.096e-06 8.192e-06)
VIN13 nreq13 0 PULSE(0 1.8 4.096e-06 20p 20p 8.192e-06 1.6384e-05)
VIN14 nreq14 0 PULSE(0 1.8 8.192e-06 20p 20p 1.6384e-05 3.2768e-05)
VIN15 nreq15 0 PULSE(0 1.8 1.6384e-05 20p 20p 3.2768e-05 6.5536e-05)
VIN16 nreq16 0 PULSE(0 1.8 3.2768e-05 20p 20p 6.5536e-05 0.000131072)
VIN17 nreq17 0 PULSE(0 1.8 6.5536e-05 20p 20p 0.000131072 0.000262144)
VIN18 nreq18 0 PULSE(0 1.8 0.000131072 20p 20p 0.000262144 0.000524288)
VIN19 nreq19 0 PULSE(0 1.8 0.000262144 20p 20p 0.000524288 0.001048576)
VIN20 nreq20 0 PULSE(0 1.8 0.000524288 20p 20p 0.001048576 0.002097152)
VIN21 nreq21 0 PULSE(0 1.8 0.001048576 20p 20p 0.002097152 0.004194304)
VIN22 nreq22 0 PULSE(0 1.8 0.002097152 20p 20p 0.004194304 0.008388608)
VIN23 nreq23 0 PULSE(0 1.8 0.004194304 20p 20p 0.008388608 0.016777216)
VIN24 nreq24 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN25 nreq25 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN26 nreq26 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN27 nen0 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN28 nen1 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN29 nen2 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN30 nen3 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN31 nen4 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN32 nen5 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN33 nen6 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN34 nen7 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN35 nen8 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN36 nen9 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN37 nen10 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN38 nen11 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN39 nen12 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN40 nen13 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN41 nen14 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN42 nen15 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN43 nen16 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN44 nen17 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN45 nen18 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN46 nen19 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN47 nen20 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN48 nen21 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN49 nen22 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN50 nen23 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN51 nen24 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN52 nen25 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN53 nen26 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
CT1 t1 0 0.1f
M1 t1 nreq0 vdd vdd pch w=2u l=180n
M2 t1 nen0 vdd vdd pch w=2u l=180n
CT2 t2 0 0.1f
M3 t1 nreq0 t2 0 nch w=1u l=180n
M4 t2 nen0 0 0 nch w=1u l=180n
M5 nw1 t1 vdd vdd pch w=2u l=180n
M6 nw1 t1 0 0 nch w=1u l=180n
Cnw1 nw1 0 2f
CT3 t3 0 0.1f
M7 t3 nreq1 vdd vdd pch w=2u l=180n
M8 t3 nen1 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M9 t3 nreq1 t4 0 nch w=1u l=180n
M10 t4 nen1 0 0 nch w=1u l=180n
M11 nw2 t3 vdd vdd pch w=2u l=180n
M12 nw2 t3 0 0 nch w=1u l=180n
Cnw2 nw2 0 2f
CT5 t5 0 0.1f
M13 t5 nreq2 vdd vdd pch w=2u l=180n
M14 t5 nen2 vdd vdd pch w=2u l=180n
CT6 t6 0 0.1f
M15 t5 nreq2 t6 0 nch w=1u l=180n
M16 t6 nen2 0 0 nch w=1u l=180n
M17 nw3 t5 vdd vdd pch w=2u l=180n
M18 nw3 t5 0 0 nch w=1u l=180n
Cnw3 nw3 0 2f
CT7 t7 0 0.1f
M19 t7 nreq3 vdd vdd pch w=2u l=180n
M20 t7 nen3 vdd vdd pch w=2u l=180n
CT8 t8 0 0.1f
M21 t7 nreq3 t8 0 nch w=1u l=180n
M22 t8 nen3 0 0 nch w=1u l=180n
M23 nw4 t7 vdd vdd pch w=2u l=180n
M24 nw4 t7 0 0 nch w=1u l=180n
Cnw4 nw4 0 2f
CT9 t9 0 0.1f
M25 t9 nreq4 vdd vdd pch w=2u l=180n
M26 t9 nen4 vdd vdd pch w=2u l=180n
CT10 t10 0 0.1f
M27 t9 nreq4 t10 0 nch w=1u l=180n
M28 t10 nen4 0 0 nch w=1u l=180n
M29 nw5 t9 vdd vdd pch w=2u l=180n
M30 nw5 t9 0 0 nch w=1u l=180n
Cnw5 nw5 0 2f
CT11 t11 0 0.1f
M31 t11 nreq5 vdd vdd pch w=2u l=180n
M32 t11 nen5 vdd vdd pch w=2u l=180n
CT12 t12 0 0.1f
M33 t11 nreq5 t12 0 nch w=1u l=180n
M34 t12 nen5 0 0 nch w=1u l=180n
M35 nw6 t11 vdd vdd pch w=2u l=180n
M36 nw6 t11 0 0 nch w=1u l=180n
Cnw6 nw6 0 2f
CT13 t13 0 0.1f
M37 t13 nreq6 vdd vdd pch w=2u l=180n
M38 t13 nen6 vdd vdd pch w=2u l=180n
CT14 t14 0 0.1f
M39 t13 nreq6 t14 0 nch w=1u l=180n
M40 t14 nen6 0 0 nch w=1u l=180n
M41 nw7 t13 vdd vdd pch w=2u l=180n
M42 nw7 t13 0 0 nch w=1u l=180n
Cnw7 nw7 0 2f
CT15 t15 0 0.1f
M43 t15 nreq7 vdd vdd pch w=2u l=180n
M44 t15 nen7 vdd vdd pch w=2u l=180n
CT16 t16 0 0.1f
M45 t15 nreq7 t16 0 nch w=1u l=180n
M46 t16 nen7 0 0 nch w=1u l=180n
M47 nw8 t15 vdd vdd pch w=2u l=180n
M48 nw8 t15 0 0 nch w=1u l=180n
Cnw8 nw8 0 2f
CT17 t17 0 0.1f
M49 t17 nreq8 vdd vdd pch w=2u l=180n
M50 t17 nen8 vdd vdd pch w=2u l=180n
CT18 t18 0 0.1f
M51 t17 nreq8 t18 0 nch w=1u l=180n
M52 t18 nen8 0 0 nch w=1u l=180n
M53 nw9 t17 vdd vdd pch w=2u l=180n
M54 nw9 t17 0 0 nch w=1u l=180n
Cnw9 nw9 0 2f
CT19 t19 0 0.1f
M55 t19 nreq9 vdd vdd pch w=2u l=180n
M56 t19 nen9 vdd vdd pch w=2u l=180n
CT20 t20 0 0.1f
M57 t19 nreq9 t20 0 nch w=1u l=180n
M58 t20 nen9 0 0 nch w=1u l=180n
M59 nw10 t19 vdd vdd pch w=2u l=180n
M60 nw10 t19 0 0 nch w=1u l=180n
Cnw10 nw10 0 2f
CT21 t21 0 0.1f
M61 t21 nreq10 vdd vdd pch w=2u l=180n
M62 t21 nen10 vdd vdd pch w=2u l=180n
CT22 t22 0 0.1f
M63 t21 nreq10 t22 0 nch w=1u l=180n
M64 t22 nen10 0 0 nch w=1u l=180n
M65 nw11 t21 vdd vdd pch w=2u l=180n
M66 nw11 t21 0 0 nch w=1u l=180n
Cnw11 nw11 0 2f
CT23 t23 0 0.1f
M67 t23 nreq11 vdd vdd pch w=2u l=180n
M68 t23 nen11 vdd vdd pch w=2u l=180n
CT24 t24 0 0.1f
M69 t23 nreq11 t24 0 nch w=1u l=180n
M70 t24 nen11 0 0 nch w=1u l=180n
M71 nw12 t23 vdd vdd pch w=2u l=180n
M72 nw12 t23 0 0 nch w=1u l=180n
Cnw12 nw12 0 2f
CT25 t25 0 0.1f
M73 t25 nreq12 vdd vdd pch w=2u l=180n
M74 t25 nen12 vdd vdd pch w=2u l=180n
CT26 t26 0 0.1f
M75 t25 nreq12 t26 0 nch w=1u l=180n
M76 t26 nen12 0 0 nch w=1u l=180n
M77 nw13 t25 vdd vdd pch w=2u l=180n
M78 nw13 t25 0 0 nch w=1u l=180n
Cnw13 nw13 0 2f
CT27 t27 0 0.1f
M79 t27 nreq13 vdd vdd pch w=2u l=180n
M80 t27 nen13 vdd vdd pch w=2u l=180n
CT28 t28 0 0.1f
M81 t27 nreq13 t28 0 nch w=1u l=180n
M82 t28 nen13 0 0 nch w=1u l=180n
M83 nw14 t27 vdd vdd pch w=2u l=180n
M84 nw14 t27 0 0 nch w=1u l=180n
Cnw14 nw14 0 2f
CT29 t29 0 0.1f
M85 t29 nreq14 vdd vdd pch w=2u l=180n
M86 t29 nen14 vdd vdd pch w=2u l=180n
CT30 t30 0 0.1f
M87 t29 nreq14 t30 0 nch w=1u l=180n
M88 t30 nen14 0 0 nch w=1u l=180n
M89 nw15 t29 vdd vdd pch w=2u l=180n
M90 nw15 t29 0 0 nch w=1u l=180n
Cnw15 nw15 0 2f
CT31 t31 0 0.1f
M91 t31 nreq15 vdd vdd pch w=2u l=180n
M92 t31 nen15 vdd vdd pch w=2u l=180n
CT32 t32 0 0.1f
M93 t31 nreq15 t32 0 nch w=1u l=180n
M94 t32 nen15 0 0 nch w=1u l=180n
M95 nw16 t31 vdd vdd pch w=2u l=180n
M96 nw16 t31 0 0 nch w=1u l=180n
Cnw16 nw16 0 2f
CT33 t33 0 0.1f
M97 t33 nreq16 vdd vdd pch w=2u l=180n
M98 t33 nen16 vdd vdd pch w=2u l=180n
CT34 t34 0 0.1f
M99 t33 nreq16 t34 0 nch w=1u l=180n
M100 t34 nen16 0 0 nch w=1u l=180n
M101 nw17 t33 vdd vdd pch w=2u l=180n
M102 nw17 t33 0 0 nch w=1u l=180n
Cnw17 nw17 0 2f
CT35 t35 0 0.1f
M103 t35 nreq17 vdd vdd pch w=2u l=180n
M104 t35 nen17 vdd vdd pch w=2u l=180n
CT36 t36 0 0.1f
M105 t35 nreq17 t36 0 nch w=1u l=180n
M106 t36 nen17 0 0 nch w=1u l=180n
M107 nw18 t35 vdd vdd pch w=2u l=180n
M108 nw18 t35 0 0 nch w=1u l=180n
Cnw18 nw18 0 2f
CT37 t37 0 0.1f
M109 t37 nreq18 vdd vdd pch w=2u l=180n
M110 t37 nen18 vdd vdd pch w=2u l=180n
CT38 t38 0 0.1f
M111 t37 nreq18 t38 0 nch w=1u l=180n
M112 t38 nen18 0 0 nch w=1u l=180n
M113 nw19 t37 vdd vdd pch w=2u l=180n
M114 nw19 t37 0 0 nch w=1u l=180n
Cnw19 nw19 0 2f
CT39 t39 0 0.1f
M115 t39 nreq19 vdd vdd pch w=2u l=180n
M116 t39 nen19 vdd vdd pch w=2u l=180n
CT40 t40 0 0.1f
M117 t39 nreq19 t40 0 nch w=1u l=180n
M118 t40 nen19 0 0 nch w=1u l=180n
M119 nw20 t39 vdd vdd pch w=2u l=180n
M120 nw20 t39 0 0 nch w=1u l=180n
Cnw20 nw20 0 2f
CT41 t41 0 0.1f
M121 t41 nreq20 vdd vdd pch w=2u l=180n
M122 t41 nen20 vdd vdd pch w=2u l=180n
CT42 t42 0 0.1f
M123 t41 nreq20 t42 0 nch w=1u l=180n
M124 t42 nen20 0 0 nch w=1u l=180n
M125 nw21 t41 vdd vdd pch w=2u l=180n
M126 nw21 t41 0 0 nch w=1u l=180n
Cnw21 nw21 0 2f
CT43 t43 0 0.1f
M127 t43 nreq21 vdd vdd pch w=2u l=180n
M128 t43 nen21 vdd vdd pch w=2u l=180n
CT44 t44 0 0.1f
M129 t43 nreq21 t44 0 nch w=1u l=180n
M130 t44 nen21 0 0 nch w=1u l=180n
M131 nw22 t43 vdd vdd pch w=2u l=180n
M132 nw22 t43 0 0 nch w=1u l=180n
Cnw22 nw22 0 2f
CT45 t45 0 0.1f
M133 t45 nreq22 vdd vdd pch w=2u l=180n
M134 t45 nen22 vdd vdd pch w=2u l=180n
CT46 t46 0 0.1f
M135 t45 nreq22 t46 0 nch w=1u l=180n
M136 t46 nen22 0 0 nch w=1u l=180n
M137 nw23 t45 vdd vdd pch w=2u l=180n
M138 nw23 t45 0 0 nch w=1u l=180n
Cnw23 nw23 0 2f
CT47 t47 0 0.1f
M139 t47 nreq23 vdd vdd pch w=2u l=180n
M140 t47 nen23 vdd vdd pch w=2u l=180n
CT48 t48 0 0.1f
M141 t47 nreq23 t48 0 nch w=1u l=180n
M142 t48 nen23 0 0 nch w=1u l=180n
M143 nw24 t47 vdd vdd pch w=2u l=180n
M144 nw24 t47 0 0 nch w=1u l=180n
Cnw24 nw24 0 2f
CT49 t49 0 0.1f
M145 t49 nreq24 vdd vdd pch w=2u l=180n
M146 t49 nen24 vdd vdd pch w=2u l=180n
CT50 t50 0 0.1f
M147 t49 nreq24 t50 0 nch w=1u l=180n
M148 t50 nen24 0 0 nch w=1u l=180n
M149 nw25 t49 vdd vdd pch w=2u l=180n
M150 nw25 t49 0 0 nch w=1u l=180n
Cnw25 nw25 0 2f
CT51 t51 0 0.1f
M151 t51 nreq25 vdd vdd pch w=2u l=180n
M152 t51 nen25 vdd vdd pch w=2u l=180n
CT52 t52 0 0.1f
M153 t51 nreq25 t52 0 nch w=1u l=180n
M154 t52 nen25 0 0 nch w=1u l=180n
M155 nw26 t51 vdd vdd pch w=2u l=180n
M156 nw26 t51 0 0 nch w=1u l=180n
Cnw26 nw26 0 2f
CT53 t53 0 0.1f
M157 t53 nreq26 vdd vdd pch w=2u l=180n
M158 t53 nen26 vdd vdd pch w=2u l=180n
CT54 t54 0 0.1f
M159 t53 nreq26 t54 0 nch w=1u l=180n
M160 t54 nen26 0 0 nch w=1u l=180n
M161 nw27 t53 vdd vdd pch w=2u l=180n
M162 nw27 t53 0 0 nch w=1u l=180n
Cnw27 nw27 0 2f
M163 nw28 nw1 vdd vdd pch w=2u l=180n
M164 nw28 nw1 0 0 nch w=1u l=180n
Cnw28 nw28 0 2f
CT55 t55 0 0.1f
M165 t55 nw2 vdd vdd pch w=2u l=180n
M166 t55 nw28 vdd vdd pch w=2u l=180n
CT56 t56 0 0.1f
M167 t55 nw2 t56 0 nch w=1u l=180n
M168 t56 nw28 0 0 nch w=1u l=180n
M169 nw29 t55 vdd vdd pch w=2u l=180n
M170 nw29 t55 0 0 nch w=1u l=180n
Cnw29 nw29 0 2f
CT57 t57 0 0.1f
M171 t57 nw1 0 0 nch w=1u l=180n
M172 t57 nw2 0 0 nch w=1u l=180n
CT58 t58 0 0.1f
M173 t58 nw1 vdd vdd pch w=2u l=180n
M174 t57 nw2 t58 vdd pch w=2u l=180n
M175 nw30 t57 vdd vdd pch w=2u l=180n
M176 nw30 t57 0 0 nch w=1u l=180n
Cnw30 nw30 0 2f
M177 nw31 nw30 vdd vdd pch w=2u l=180n
M178 nw31 nw30 0 0 nch w=1u l=180n
Cnw31 nw31 0 2f
CT59 t59 0 0.1f
M179 t59 nw3 vdd vdd pch w=2u l=180n
M180 t59 nw31 vdd vdd pch w=2u l=180n
CT60 t60 0 0.1f
M181 t59 nw3 t60 0 nch w=1u l=180n
M182 t60 nw31 0 0 nch w=1u l=180n
M183 nw32 t59 vdd vdd pch w=2u l=180n
M184 nw32 t59 0 0 nch w=1u l=180n
Cnw32 nw32 0 2f
CT61 t61 0 0.1f
M185 t61 nw30 0 0 nch w=1u l=180n
M186 t61 nw3 0 0 nch w=1u l=180n
CT62 t62 0 0.1f
M187 t62 nw30 vdd vdd pch w=2u l=180n
M188 t61 nw3 t62 vdd pch w=2u l=180n
M189 nw33 t61 vdd vdd pch w=2u l=180n
M190 nw33 t61 0 0 nch w=1u l=180n
Cnw33 nw33 0 2f
M191 nw34 nw33 vdd vdd pch w=2u l=180n
M192 nw34 nw33 0 0 nch w=1u l=180n
Cnw34 nw34 0 2f
CT63 t63 0 0.1f
M193 t63 nw4 vdd vdd pch w=2u l=180n
M194 t63 nw34 vdd vdd pch w=2u l=180n
CT64 t64 0 0.1f
M195 t63 nw4 t64 0 nch w=1u l=180n
M196 t64 nw34 0 0 nch w=1u l=180n
M197 nw35 t63 vdd vdd pch w=2u l=180n
M198 nw35 t63 0 0 nch w=1u l=180n
Cnw35 nw35 0 2f
CT65 t65 0 0.1f
M199 t65 nw33 0 0 nch w=1u l=180n
M200 t65 nw4 0 0 nch w=1u l=180n
CT66 t66 0 0.1f
M201 t66 nw33 vdd vdd pch w=2u l=180n
M202 t65 nw4 t66 vdd pch w=2u l=180n
M203 nw36 t65 vdd vdd pch w=2u l=180n
M204 nw36 t65 0 0 nch w=1u l=180n
Cnw36 nw36 0 2f
M205 nw37 nw36 vdd vdd pch w=2u l=180n
M206 nw37 nw36 0 0 nch w=1u l=180n
Cnw37 nw37 0 2f
CT67 t67 0 0.1f
M207 t67 nw5 vdd vdd pch w=2u l=180n
M208 t67 nw37 vdd vdd pch w=2u l=180n
CT68 t68 0 0.1f
M209 t67 nw5 t68 0 nch w=1u l=180n
M210 t68 nw37 0 0 nch w=1u l=180n
M211 nw38 t67 vdd vdd pch w=2u l=180n
M212 nw38 t67 0 0 nch w=1u l=180n
Cnw38 nw38 0 2f
CT69 t69 0 0.1f
M213 t69 nw36 0 0 nch w=1u l=180n
M214 t69 nw5 0 0 nch w=1u l=180n
CT70 t70 0 0.1f
M215 t70 nw36 vdd vdd pch w=2u l=180n
M216 t69 nw5 t70 vdd pch w=2u l=180n
M217 nw39 t69 vdd vdd pch w=2u l=180n
M218 nw39 t69 0 0 nch w=1u l=180n
Cnw39 nw39 0 2f
M219 nw40 nw39 vdd vdd pch w=2u l=180n
M220 nw40 nw39 0 0 nch w=1u l=180n
Cnw40 nw40 0 2f
CT71 t71 0 0.1f
M221 t71 nw6 vdd vdd pch w=2u l=180n
M222 t71 nw40 vdd vdd pch w=2u l=180n
CT72 t72 0 0.1f
M223 t71 nw6 t72 0 nch w=1u l=180n
M224 t72 nw40 0 0 nch w=1u l=180n
M225 nw41 t71 vdd vdd pch w=2u l=180n
M226 nw41 t71 0 0 nch w=1u l=180n
Cnw41 nw41 0 2f
CT73 t73 0 0.1f
M227 t73 nw39 0 0 nch w=1u l=180n
M228 t73 nw6 0 0 nch w=1u l=180n
CT74 t74 0 0.1f
M229 t74 nw39 vdd vdd pch w=2u l=180n
M230 t73 nw6 t74 vdd pch w=2u l=180n
M231 nw42 t73 vdd vdd pch w=2u l=180n
M232 nw42 t73 0 0 nch w=1u l=180n
Cnw42 nw42 0 2f
M233 nw43 nw42 vdd vdd pch w=2u l=180n
M234 nw43 nw42 0 0 nch w=1u l=180n
Cnw43 nw43 0 2f
CT75 t75 0 0.1f
M235 t75 nw7 vdd vdd pch w=2u l=180n
M236 t75 nw43 vdd vdd pch w=2u l=180n
CT76 t76 0 0.1f
M237 t75 nw7 t76 0 nch w=1u l=180n
M238 t76 nw43 0 0 nch w=1u l=180n
M239 nw44 t75 vdd vdd pch w=2u l=180n
M240 nw44 t75 0 0 nch w=1u l=180n
Cnw44 nw44 0 2f
CT77 t77 0 0.1f
M241 t77 nw42 0 0 nch w=1u l=180n
M242 t77 nw7 0 0 nch w=1u l=180n
CT78 t78 0 0.1f
M243 t78 nw42 vdd vdd pch w=2u l=180n
M244 t77 nw7 t78 vdd pch w=2u l=180n
M245 nw45 t77 vdd vdd pch w=2u l=180n
M246 nw45 t77 0 0 nch w=1u l=180n
Cnw45 nw45 0 2f
M247 nw46 nw45 vdd vdd pch w=2u l=180n
M248 nw46 nw45 0 0 nch w=1u l=180n
Cnw46 nw46 0 2f
CT79 t79 0 0.1f
M249 t79 nw8 vdd vdd pch w=2u l=180n
M250 t79 nw46 vdd vdd pch w=2u l=180n
CT80 t80 0 0.1f
M251 t79 nw8 t80 0 nch w=1u l=180n
M252 t80 nw46 0 0 nch w=1u l=180n
M253 nw47 t79 vdd vdd pch w=2u l=180n
M254 nw47 t79 0 0 nch w=1u l=180n
Cnw47 nw47 0 2f
CT81 t81 0 0.1f
M255 t81 nw45 0 0 nch w=1u l=180n
M256 t81 nw8 0 0 nch w=1u l=180n
CT82 t82 0 0.1f
M257 t82 nw45 vdd vdd pch w=2u l=180n
M258 t81 nw8 t82 vdd pch w=2u l=180n
M259 nw48 t81 vdd vdd pch w=2u l=180n
M260 nw48 t81 0 0 nch w=1u l=180n
Cnw48 nw48 0 2f
M261 nw49 nw48 vdd vdd pch w=2u l=180n
M262 nw49 nw48 0 0 nch w=1u l=180n
Cnw49 nw49 0 2f
CT83 t83 0 0.1f
M263 t83 nw9 vdd vdd pch w=2u l=180n
M264 t83 nw49 vdd vdd pch w=2u l=180n
CT84 t84 0 0.1f
M265 t83 nw9 t84 0 nch w=1u l=180n
M266 t84 nw49 0 0 nch w=1u l=180n
M267 nw50 t83 vdd vdd pch w=2u l=180n
M268 nw50 t83 0 0 nch w=1u l=180n
Cnw50 nw50 0 2f
CT85 t85 0 0.1f
M269 t85 nw48 0 0 nch w=1u l=180n
M270 t85 nw9 0 0 nch w=1u l=180n
CT86 t86 0 0.1f
M271 t86 nw48 vdd vdd pch w=2u l=180n
M272 t85 nw9 t86 vdd pch w=2u l=180n
M273 nw51 t85 vdd vdd pch w=2u l=180n
M274 nw51 t85 0 0 nch w=1u l=180n
Cnw51 nw51 0 2f
M275 nw52 nw51 vdd vdd pch w=2u l=180n
M276 nw52 nw51 0 0 nch w=1u l=180n
Cnw52 nw52 0 2f
CT87 t87 0 0.1f
M277 t87 nw10 vdd vdd pch w=2u l=180n
M278 t87 nw52 vdd vdd pch w=2u l=180n
CT88 t88 0 0.1f
M279 t87 nw10 t88 0 nch w=1u l=180n
M280 t88 nw52 0 0 nch w=1u l=180n
M281 nw53 t87 vdd vdd pch w=2u l=180n
M282 nw53 t87 0 0 nch w=1u l=180n
Cnw53 nw53 0 2f
CT89 t89 0 0.1f
M283 t89 nw51 0 0 nch w=1u l=180n
M284 t89 nw10 0 0 nch w=1u l=180n
CT90 t90 0 0.1f
M285 t90 nw51 vdd vdd pch w=2u l=180n
M286 t89 nw10 t90 vdd pch w=2u l=180n
M287 nw54 t89 vdd vdd pch w=2u l=180n
M288 nw54 t89 0 0 nch w=1u l=180n
Cnw54 nw54 0 2f
M289 nw55 nw54 vdd vdd pch w=2u l=180n
M290 nw55 nw54 0 0 nch w=1u l=180n
Cnw55 nw55 0 2f
CT91 t91 0 0.1f
M291 t91 nw11 vdd vdd pch w=2u l=180n
M292 t91 nw55 vdd vdd pch w=2u l=180n
CT92 t92 0 0.1f
M293 t91 nw11 t92 0 nch w=1u l=180n
M294 t92 nw55 0 0 nch w=1u l=180n
M295 nw56 t91 vdd vdd pch w=2u l=180n
M296 nw56 t91 0 0 nch w=1u l=180n
Cnw56 nw56 0 2f
CT93 t93 0 0.1f
M297 t93 nw54 0 0 nch w=1u l=180n
M298 t93 nw11 0 0 nch w=1u l=180n
CT94 t94 0 0.1f
M299 t94 nw54 vdd vdd pch w=2u l=180n
M300 t93 nw11 t94 vdd pch w=2u l=180n
M301 nw57 t93 vdd vdd pch w=2u l=180n
M302 nw57 t93 0 0 nch w=1u l=180n
Cnw57 nw57 0 2f
M303 nw58 nw57 vdd vdd pch w=2u l=180n
M304 nw58 nw57 0 0 nch w=1u l=180n
Cnw58 nw58 0 2f
CT95 t95 0 0.1f
M305 t95 nw12 vdd vdd pch w=2u l=180n
M306 t95 nw58 vdd vdd pch w=2u l=180n
CT96 t96 0 0.1f
M307 t95 nw12 t96 0 nch w=1u l=180n
M308 t96 nw58 0 0 nch w=1u l=180n
M309 nw59 t95 vdd vdd pch w=2u l=180n
M310 nw59 t95 0 0 nch w=1u l=180n
Cnw59 nw59 0 2f
CT97 t97 0 0.1f
M311 t97 nw57 0 0 nch w=1u l=180n
M312 t97 nw12 0 0 nch w=1u l=180n
CT98 t98 0 0.1f
M313 t98 nw57 vdd vdd pch w=2u l=180n
M314 t97 nw12 t98 vdd pch w=2u l=180n
M315 nw60 t97 vdd vdd pch w=2u l=180n
M316 nw60 t97 0 0 nch w=1u l=180n
Cnw60 nw60 0 2f
M317 nw61 nw60 vdd vdd pch w=2u l=180n
M318 nw61 nw60 0 0 nch w=1u l=180n
Cnw61 nw61 0 2f
CT99 t99 0 0.1f
M319 t99 nw13 vdd vdd pch w=2u l=180n
M320 t99 nw61 vdd vdd pch w=2u l=180n
CT100 t100 0 0.1f
M321 t99 nw13 t100 0 nch w=1u l=180n
M322 t100 nw61 0 0 nch w=1u l=180n
M323 nw62 t99 vdd vdd pch w=2u l=180n
M324 nw62 t99 0 0 nch w=1u l=180n
Cnw62 nw62 0 2f
CT101 t101 0 0.1f
M325 t101 nw60 0 0 nch w=1u l=180n
M326 t101 nw13 0 0 nch w=1u l=180n
CT102 t102 0 0.1f
M327 t102 nw60 vdd vdd pch w=2u l=180n
M328 t101 nw13 t102 vdd pch w=2u l=180n
M329 nw63 t101 vdd vdd pch w=2u l=180n
M330 nw63 t101 0 0 nch w=1u l=180n
Cnw63 nw63 0 2f
M331 nw64 nw63 vdd vdd pch w=2u l=180n
M332 nw64 nw63 0 0 nch w=1u l=180n
Cnw64 nw64 0 2f
CT103 t103 0 0.1f
M333 t103 nw14 vdd vdd pch w=2u l=180n
M334 t103 nw64 vdd vdd pch w=2u l=180n
CT104 t104 0 0.1f
M335 t103 nw14 t104 0 nch w=1u l=180n
M336 t104 nw64 0 0 nch w=1u l=180n
M337 nw65 t103 vdd vdd pch w=2u l=180n
M338 nw65 t103 0 0 nch w=1u l=180n
Cnw65 nw65 0 2f
CT105 t105 0 0.1f
M339 t105 nw63 0 0 nch w=1u l=180n
M340 t105 nw14 0 0 nch w=1u l=180n
CT106 t106 0 0.1f
M341 t106 nw63 vdd vdd pch w=2u l=180n
M342 t105 nw14 t106 vdd pch w=2u l=180n
M343 nw66 t105 vdd vdd pch w=2u l=180n
M344 nw66 t105 0 0 nch w=1u l=180n
Cnw66 nw66 0 2f
M345 nw67 nw66 vdd vdd pch w=2u l=180n
M346 nw67 nw66 0 0 nch w=1u l=180n
Cnw67 nw67 0 2f
CT107 t107 0 0.1f
M347 t107 nw15 vdd vdd pch w=2u l=180n
M348 t107 nw67 vdd vdd pch w=2u l=180n
CT108 t108 0 0.1f
M349 t107 nw15 t108 0 nch w=1u l=180n
M350 t108 nw67 0 0 nch w=1u l=180n
M351 nw68 t107 vdd vdd pch w=2u l=180n
M352 nw68 t107 0 0 nch w=1u l=180n
Cnw68 nw68 0 2f
CT109 t109 0 0.1f
M353 t109 nw66 0 0 nch w=1u l=180n
M354 t109 nw15 0 0 nch w=1u l=180n
CT110 t110 0 0.1f
M355 t110 nw66 vdd vdd pch w=2u l=180n
M356 t109 nw15 t110 vdd pch w=2u l=180n
M357 nw69 t109 vdd vdd pch w=2u l=180n
M358 nw69 t109 0 0 nch w=1u l=180n
Cnw69 nw69 0 2f
M359 nw70 nw69 vdd vdd pch w=2u l=180n
M360 nw70 nw69 0 0 nch w=1u l=180n
Cnw70 nw70 0 2f
CT111 t111 0 0.1f
M361 t111 nw16 vdd vdd pch w=2u l=180n
M362 t111 nw70 vdd vdd pch w=2u l=180n
CT112 t112 0 0.1f
M363 t111 nw16 t112 0 nch w=1u l=180n
M364 t112 nw70 0 0 nch w=1u l=180n
M365 nw71 t111 vdd vdd pch w=2u l=180n
M366 nw71 t111 0 0 nch w=1u l=180n
Cnw71 nw71 0 2f
CT113 t113 0 0.1f
M367 t113 nw69 0 0 nch w=1u l=180n
M368 t113 nw16 0 0 nch w=1u l=180n
CT114 t114 0 0.1f
M369 t114 nw69 vdd vdd pch w=2u l=180n
M370 t113 nw16 t114 vdd pch w=2u l=180n
M371 nw72 t113 vdd vdd pch w=2u l=180n
M372 nw72 t113 0 0 nch w=1u l=180n
Cnw72 nw72 0 2f
M373 nw73 nw72 vdd vdd pch w=2u l=180n
M374 nw73 nw72 0 0 nch w=1u l=180n
Cnw73 nw73 0 2f
CT115 t115 0 0.1f
M375 t115 nw17 vdd vdd pch w=2u l=180n
M376 t115 nw73 vdd vdd pch w=2u l=180n
CT116 t116 0 0.1f
M377 t115 nw17 t116 0 nch w=1u l=180n
M378 t116 nw73 0 0 nch w=1u l=180n
M379 nw74 t115 vdd vdd pch w=2u l=180n
M380 nw74 t115 0 0 nch w=1u l=180n
Cnw74 nw74 0 2f
CT117 t117 0 0.1f
M381 t117 nw72 0 0 nch w=1u l=180n
M382 t117 nw17 0 0 nch w=1u l=180n
CT118 t118 0 0.1f
M383 t118 nw72 vdd vdd pch w=2u l=180n
M384 t117 nw17 t118 vdd pch w=2u l=180n
M385 nw75 t117 vdd vdd pch w=2u l=180n
M386 nw75 t117 0 0 nch w=1u l=180n
Cnw75 nw75 0 2f
M387 nw76 nw75 vdd vdd pch w=2u l=180n
M388 nw76 nw75 0 0 nch w=1u l=180n
Cnw76 nw76 0 2f
CT119 t119 0 0.1f
M389 t119 nw18 vdd vdd pch w=2u l=180n
M390 t119 nw76 vdd vdd pch w=2u l=180n
CT120 t120 0 0.1f
M391 t119 nw18 t120 0 nch w=1u l=180n
M392 t120 nw76 0 0 nch w=1u l=180n
M393 nw77 t119 vdd vdd pch w=2u l=180n
M394 nw77 t119 0 0 nch w=1u l=180n
Cnw77 nw77 0 2f
CT121 t121 0 0.1f
M395 t121 nw75 0 0 nch w=1u l=180n
M396 t121 nw18 0 0 nch w=1u l=180n
CT122 t122 0 0.1f
M397 t122 nw75 vdd vdd pch w=2u l=180n
M398 t121 nw18 t122 vdd pch w=2u l=180n
M399 nw78 t121 vdd vdd pch w=2u l=180n
M400 nw78 t121 0 0 nch w=1u l=180n
Cnw78 nw78 0 2f
M401 nw79 nw78 vdd vdd pch w=2u l=180n
M402 nw79 nw78 0 0 nch w=1u l=180n
Cnw79 nw79 0 2f
CT123 t123 0 0.1f
M403 t123 nw19 vdd vdd pch w=2u l=180n
M404 t123 nw79 vdd vdd pch w=2u l=180n
CT124 t124 0 0.1f
M405 t123 nw19 t124 0 nch w=1u l=180n
M406 t124 nw79 0 0 nch w=1u l=180n
M407 nw80 t123 vdd vdd pch w=2u l=180n
M408 nw80 t123 0 0 nch w=1u l=180n
Cnw80 nw80 0 2f
CT125 t125 0 0.1f
M409 t125 nw78 0 0 nch w=1u l=180n
M410 t125 nw19 0 0 nch w=1u l=180n
CT126 t126 0 0.1f
M411 t126 nw78 vdd vdd pch w=2u l=180n
M412 t125 nw19 t126 vdd pch w=2u l=180n
M413 nw81 t125 vdd vdd pch w=2u l=180n
M414 nw81 t125 0 0 nch w=1u l=180n
Cnw81 nw81 0 2f
M415 nw82 nw81 vdd vdd pch w=2u l=180n
M416 nw82 nw81 0 0 nch w=1u l=180n
Cnw82 nw82 0 2f
CT127 t127 0 0.1f
M417 t127 nw20 vdd vdd pch w=2u l=180n
M418 t127 nw82 vdd vdd pch w=2u l=180n
CT128 t128 0 0.1f
M419 t127 nw20 t128 0 nch w=1u l=180n
M420 t128 nw82 0 0 nch w=1u l=180n
M421 nw83 t127 vdd vdd pch w=2u l=180n
M422 nw83 t127 0 0 nch w=1u l=180n
Cnw83 nw83 0 2f
CT129 t129 0 0.1f
M423 t129 nw81 0 0 nch w=1u l=180n
M424 t129 nw20 0 0 nch w=1u l=180n
CT130 t130 0 0.1f
M425 t130 nw81 vdd vdd pch w=2u l=180n
M426 t129 nw20 t130 vdd pch w=2u l=180n
M427 nw84 t129 vdd vdd pch w=2u l=180n
M428 nw84 t129 0 0 nch w=1u l=180n
Cnw84 nw84 0 2f
M429 nw85 nw84 vdd vdd pch w=2u l=180n
M430 nw85 nw84 0 0 nch w=1u l=180n
Cnw85 nw85 0 2f
CT131 t131 0 0.1f
M431 t131 nw21 vdd vdd pch w=2u l=180n
M432 t131 nw85 vdd vdd pch w=2u l=180n
CT132 t132 0 0.1f
M433 t131 nw21 t132 0 nch w=1u l=180n
M434 t132 nw85 0 0 nch w=1u l=180n
M435 nw86 t131 vdd vdd pch w=2u l=180n
M436 nw86 t131 0 0 nch w=1u l=180n
Cnw86 nw86 0 2f
CT133 t133 0 0.1f
M437 t133 nw84 0 0 nch w=1u l=180n
M438 t133 nw21 0 0 nch w=1u l=180n
CT134 t134 0 0.1f
M439 t134 nw84 vdd vdd pch w=2u l=180n
M440 t133 nw21 t134 vdd pch w=2u l=180n
M441 nw87 t133 vdd vdd pch w=2u l=180n
M442 nw87 t133 0 0 nch w=1u l=180n
Cnw87 nw87 0 2f
M443 nw88 nw87 vdd vdd pch w=2u l=180n
M444 nw88 nw87 0 0 nch w=1u l=180n
Cnw88 nw88 0 2f
CT135 t135 0 0.1f
M445 t135 nw22 vdd vdd pch w=2u l=180n
M446 t135 nw88 vdd vdd pch w=2u l=180n
CT136 t136 0 0.1f
M447 t135 nw22 t136 0 nch w=1u l=180n
M448 t136 nw88 0 0 nch w=1u l=180n
M449 nw89 t135 vdd vdd pch w=2u l=180n
M450 nw89 t135 0 0 nch w=1u l=180n
Cnw89 nw89 0 2f
CT137 t137 0 0.1f
M451 t137 nw87 0 0 nch w=1u l=180n
M452 t137 nw22 0 0 nch w=1u l=180n
CT138 t138 0 0.1f
M453 t138 nw87 vdd vdd pch w=2u l=180n
M454 t137 nw22 t138 vdd pch w=2u l=180n
M455 nw90 t137 vdd vdd pch w=2u l=180n
M456 nw90 t137 0 0 nch w=1u l=180n
Cnw90 nw90 0 2f
M457 nw91 nw90 vdd vdd pch w=2u l=180n
M458 nw91 nw90 0 0 nch w=1u l=180n
Cnw91 nw91 0 2f
CT139 t139 0 0.1f
M459 t139 nw23 vdd vdd pch w=2u l=180n
M460 t139 nw91 vdd vdd pch w=2u l=180n
CT140 t140 0 0.1f
M461 t139 nw23 t140 0 nch w=1u l=180n
M462 t140 nw91 0 0 nch w=1u l=180n
M463 nw92 t139 vdd vdd pch w=2u l=180n
M464 nw92 t139 0 0 nch w=1u l=180n
Cnw92 nw92 0 2f
CT141 t141 0 0.1f
M465 t141 nw90 0 0 nch w=1u l=180n
M466 t141 nw23 0 0 nch w=1u l=180n
CT142 t142 0 0.1f
M467 t142 nw90 vdd vdd pch w=2u l=180n
M468 t141 nw23 t142 vdd pch w=2u l=180n
M469 nw93 t141 vdd vdd pch w=2u l=180n
M470 nw93 t141 0 0 nch w=1u l=180n
Cnw93 nw93 0 2f
M471 nw94 nw93 vdd vdd pch w=2u l=180n
M472 nw94 nw93 0 0 nch w=1u l=180n
Cnw94 nw94 0 2f
CT143 t143 0 0.1f
M473 t143 nw24 vdd vdd pch w=2u l=180n
M474 t143 nw94 vdd vdd pch w=2u l=180n
CT144 t144 0 0.1f
M475 t143 nw24 t144 0 nch w=1u l=180n
M476 t144 nw94 0 0 nch w=1u l=180n
M477 nw95 t143 vdd vdd pch w=2u l=180n
M478 nw95 t143 0 0 nch w=1u l=180n
Cnw95 nw95 0 2f
CT145 t145 0 0.1f
M479 t145 nw93 0 0 nch w=1u l=180n
M480 t145 nw24 0 0 nch w=1u l=180n
CT146 t146 0 0.1f
M481 t146 nw93 vdd vdd pch w=2u l=180n
M482 t145 nw24 t146 vdd pch w=2u l=180n
M483 nw96 t145 vdd vdd pch w=2u l=180n
M484 nw96 t145 0 0 nch w=1u l=180n
Cnw96 nw96 0 2f
M485 nw97 nw96 vdd vdd pch w=2u l=180n
M486 nw97 nw96 0 0 nch w=1u l=180n
Cnw97 nw97 0 2f
CT147 t147 0 0.1f
M487 t147 nw25 vdd vdd pch w=2u l=180n
M488 t147 nw97 vdd vdd pch w=2u l=180n
CT148 t148 0 0.1f
M489 t147 nw25 t148 0 nch w=1u l=180n
M490 t148 nw97 0 0 nch w=1u l=180n
M491 nw98 t147 vdd vdd pch w=2u l=180n
M492 nw98 t147 0 0 nch w=1u l=180n
Cnw98 nw98 0 2f
CT149 t149 0 0.1f
M493 t149 nw96 0 0 nch w=1u l=180n
M494 t149 nw25 0 0 nch w=1u l=180n
CT150 t150 0 0.1f
M495 t150 nw96 vdd vdd pch w=2u l=180n
M496 t149 nw25 t150 vdd pch w=2u l=180n
M497 nw99 t149 vdd vdd pch w=2u l=180n
M498 nw99 t149 0 0 nch w=1u l=180n
Cnw99 nw99 0 2f
M499 nw100 nw99 vdd vdd pch w=2u l=180n
M500 nw100 nw99 0 0 nch w=1u l=180n
Cnw100 nw100 0 2f
CT151 t151 0 0.1f
M501 t151 nw26 vdd vdd pch w=2u l=180n
M502 t151 nw100 vdd vdd pch w=2u l=180n
CT152 t152 0 0.1f
M503 t151 nw26 t152 0 nch w=1u l=180n
M504 t152 nw100 0 0 nch w=1u l=180n
M505 nw101 t151 vdd vdd pch w=2u l=180n
M506 nw101 t151 0 0 nch w=1u l=180n
Cnw101 nw101 0 2f
CT153 t153 0 0.1f
M507 t153 nw99 0 0 nch w=1u l=180n
M508 t153 nw26 0 0 nch w=1u l=180n
CT154 t154 0 0.1f
M509 t154 nw99 vdd vdd pch w=2u l=180n
M510 t153 nw26 t154 vdd pch w=2u l=180n
M511 nw102 t153 vdd vdd pch w=2u l=180n
M512 nw102 t153 0 0 nch w=1u l=180n
Cnw102 nw102 0 2f
M513 nw103 nw102 vdd vdd pch w=2u l=180n
M514 nw103 nw102 0 0 nch w=1u l=180n
Cnw103 nw103 0 2f
CT155 t155 0 0.1f
M515 t155 nw27 vdd vdd pch w=2u l=180n
M516 t155 nw103 vdd vdd pch w=2u l=180n
CT156 t156 0 0.1f
M517 t155 nw27 t156 0 nch w=1u l=180n
M518 t156 nw103 0 0 nch w=1u l=180n
M519 nw104 t155 vdd vdd pch w=2u l=180n
M520 nw104 t155 0 0 nch w=1u l=180n
Cnw104 nw104 0 2f
CT157 t157 0 0.1f
M521 t157 nw102 0 0 nch w=1u l=180n
M522 t157 nw27 0 0 nch w=1u l=180n
CT158 t158 0 0.1f
M523 t158 nw102 vdd vdd pch w=2u l=180n
M524 t157 nw27 t158 vdd pch w=2u l=180n
M525 nw105 t157 vdd vdd pch w=2u l=180n
M526 nw105 t157 0 0 nch w=1u l=180n
Cnw105 nw105 0 2f
CT159 t159 0 0.1f
M527 t159 nw29 0 0 nch w=1u l=180n
M528 t159 nw35 0 0 nch w=1u l=180n
M529 t159 nw41 0 0 nch w=1u l=180n
M530 t159 nw47 0 0 nch w=1u l=180n
CT160 t160 0 0.1f
M531 t160 nw29 vdd vdd pch w=2u l=180n
CT161 t161 0 0.1f
M532 t161 nw35 t160 vdd pch w=2u l=180n
CT162 t162 0 0.1f
M533 t162 nw41 t161 vdd pch w=2u l=180n
M534 t159 nw47 t162 vdd pch w=2u l=180n
M535 nw106 t159 vdd vdd pch w=2u l=180n
M536 nw106 t159 0 0 nch w=1u l=180n
Cnw106 nw106 0 2f
CT163 t163 0 0.1f
M537 t163 nw53 0 0 nch w=1u l=180n
M538 t163 nw59 0 0 nch w=1u l=180n
M539 t163 nw65 0 0 nch w=1u l=180n
M540 t163 nw71 0 0 nch w=1u l=180n
CT164 t164 0 0.1f
M541 t164 nw53 vdd vdd pch w=2u l=180n
CT165 t165 0 0.1f
M542 t165 nw59 t164 vdd pch w=2u l=180n
CT166 t166 0 0.1f
M543 t166 nw65 t165 vdd pch w=2u l=180n
M544 t163 nw71 t166 vdd pch w=2u l=180n
M545 nw107 t163 vdd vdd pch w=2u l=180n
M546 nw107 t163 0 0 nch w=1u l=180n
Cnw107 nw107 0 2f
CT167 t167 0 0.1f
M547 t167 nw77 0 0 nch w=1u l=180n
M548 t167 nw83 0 0 nch w=1u l=180n
M549 t167 nw89 0 0 nch w=1u l=180n
M550 t167 nw95 0 0 nch w=1u l=180n
CT168 t168 0 0.1f
M551 t168 nw77 vdd vdd pch w=2u l=180n
CT169 t169 0 0.1f
M552 t169 nw83 t168 vdd pch w=2u l=180n
CT170 t170 0 0.1f
M553 t170 nw89 t169 vdd pch w=2u l=180n
M554 t167 nw95 t170 vdd pch w=2u l=180n
M555 nw108 t167 vdd vdd pch w=2u l=180n
M556 nw108 t167 0 0 nch w=1u l=180n
Cnw108 nw108 0 2f
CT171 t171 0 0.1f
M557 t171 nw106 0 0 nch w=1u l=180n
M558 t171 nw107 0 0 nch w=1u l=180n
M559 t171 nw108 0 0 nch w=1u l=180n
M560 t171 nw101 0 0 nch w=1u l=180n
CT172 t172 0 0.1f
M561 t172 nw106 vdd vdd pch w=2u l=180n
CT173 t173 0 0.1f
M562 t173 nw107 t172 vdd pch w=2u l=180n
CT174 t174 0 0.1f
M563 t174 nw108 t173 vdd pch w=2u l=180n
M564 t171 nw101 t174 vdd pch w=2u l=180n
M565 nw109 t171 vdd vdd pch w=2u l=180n
M566 nw109 t171 0 0 nch w=1u l=180n
Cnw109 nw109 0 2f
CT175 t175 0 0.1f
M567 t175 nw109 vdd vdd pch w=2u l=180n
M568 t175 nw109 0 0 nch w=1u l=180n
M569 nidx0 t175 vdd vdd pch w=2u l=180n
M570 nidx0 t175 0 0 nch w=1u l=180n
Cnidx0 nidx0 0 2f
CT176 t176 0 0.1f
M571 t176 nw32 0 0 nch w=1u l=180n
M572 t176 nw35 0 0 nch w=1u l=180n
M573 t176 nw44 0 0 nch w=1u l=180n
M574 t176 nw47 0 0 nch w=1u l=180n
CT177 t177 0 0.1f
M575 t177 nw32 vdd vdd pch w=2u l=180n
CT178 t178 0 0.1f
M576 t178 nw35 t177 vdd pch w=2u l=180n
CT179 t179 0 0.1f
M577 t179 nw44 t178 vdd pch w=2u l=180n
M578 t176 nw47 t179 vdd pch w=2u l=180n
M579 nw111 t176 vdd vdd pch w=2u l=180n
M580 nw111 t176 0 0 nch w=1u l=180n
Cnw111 nw111 0 2f
CT180 t180 0 0.1f
M581 t180 nw56 0 0 nch w=1u l=180n
M582 t180 nw59 0 0 nch w=1u l=180n
M583 t180 nw68 0 0 nch w=1u l=180n
M584 t180 nw71 0 0 nch w=1u l=180n
CT181 t181 0 0.1f
M585 t181 nw56 vdd vdd pch w=2u l=180n
CT182 t182 0 0.1f
M586 t182 nw59 t181 vdd pch w=2u l=180n
CT183 t183 0 0.1f
M587 t183 nw68 t182 vdd pch w=2u l=180n
M588 t180 nw71 t183 vdd pch w=2u l=180n
M589 nw112 t180 vdd vdd pch w=2u l=180n
M590 nw112 t180 0 0 nch w=1u l=180n
Cnw112 nw112 0 2f
CT184 t184 0 0.1f
M591 t184 nw80 0 0 nch w=1u l=180n
M592 t184 nw83 0 0 nch w=1u l=180n
M593 t184 nw92 0 0 nch w=1u l=180n
M594 t184 nw95 0 0 nch w=1u l=180n
CT185 t185 0 0.1f
M595 t185 nw80 vdd vdd pch w=2u l=180n
CT186 t186 0 0.1f
M596 t186 nw83 t185 vdd pch w=2u l=180n
CT187 t187 0 0.1f
M597 t187 nw92 t186 vdd pch w=2u l=180n
M598 t184 nw95 t187 vdd pch w=2u l=180n
M599 nw113 t184 vdd vdd pch w=2u l=180n
M600 nw113 t184 0 0 nch w=1u l=180n
Cnw113 nw113 0 2f
CT188 t188 0 0.1f
M601 t188 nw111 0 0 nch w=1u l=180n
M602 t188 nw112 0 0 nch w=1u l=180n
M603 t188 nw113 0 0 nch w=1u l=180n
M604 t188 nw104 0 0 nch w=1u l=180n
CT189 t189 0 0.1f
M605 t189 nw111 vdd vdd pch w=2u l=180n
CT190 t190 0 0.1f
M606 t190 nw112 t189 vdd pch w=2u l=180n
CT191 t191 0 0.1f
M607 t191 nw113 t190 vdd pch w=2u l=180n
M608 t188 nw104 t191 vdd pch w=2u l=180n
M609 nw114 t188 vdd vdd pch w=2u l=180n
M610 nw114 t188 0 0 nch w=1u l=180n
Cnw114 nw114 0 2f
CT192 t192 0 0.1f
M611 t192 nw114 vdd vdd pch w=2u l=180n
M612 t192 nw114 0 0 nch w=1u l=180n
M613 nidx1 t192 vdd vdd pch w=2u l=180n
M614 nidx1 t192 0 0 nch w=1u l=180n
Cnidx1 nidx1 0 2f
CT193 t193 0 0.1f
M615 t193 nw38 0 0 nch w=1u l=180n
M616 t193 nw41 0 0 nch w=1u l=180n
M617 t193 nw44 0 0 nch w=1u l=180n
M618 t193 nw47 0 0 nch w=1u l=180n
CT194 t194 0 0.1f
M619 t194 nw38 vdd vdd pch w=2u l=180n
CT195 t195 0 0.1f
M620 t195 nw41 t194 vdd pch w=2u l=180n
CT196 t196 0 0.1f
M621 t196 nw44 t195 vdd pch w=2u l=180n
M622 t193 nw47 t196 vdd pch w=2u l=180n
M623 nw116 t193 vdd vdd pch w=2u l=180n
M624 nw116 t193 0 0 nch w=1u l=180n
Cnw116 nw116 0 2f
CT197 t197 0 0.1f
M625 t197 nw62 0 0 nch w=1u l=180n
M626 t197 nw65 0 0 nch w=1u l=180n
M627 t197 nw68 0 0 nch w=1u l=180n
M628 t197 nw71 0 0 nch w=1u l=180n
CT198 t198 0 0.1f
M629 t198 nw62 vdd vdd pch w=2u l=180n
CT199 t199 0 0.1f
M630 t199 nw65 t198 vdd pch w=2u l=180n
CT200 t200 0 0.1f
M631 t200 nw68 t199 vdd pch w=2u l=180n
M632 t197 nw71 t200 vdd pch w=2u l=180n
M633 nw117 t197 vdd vdd pch w=2u l=180n
M634 nw117 t197 0 0 nch w=1u l=180n
Cnw117 nw117 0 2f
CT201 t201 0 0.1f
M635 t201 nw86 0 0 nch w=1u l=180n
M636 t201 nw89 0 0 nch w=1u l=180n
M637 t201 nw92 0 0 nch w=1u l=180n
M638 t201 nw95 0 0 nch w=1u l=180n
CT202 t202 0 0.1f
M639 t202 nw86 vdd vdd pch w=2u l=180n
CT203 t203 0 0.1f
M640 t203 nw89 t202 vdd pch w=2u l=180n
CT204 t204 0 0.1f
M641 t204 nw92 t203 vdd pch w=2u l=180n
M642 t201 nw95 t204 vdd pch w=2u l=180n
M643 nw118 t201 vdd vdd pch w=2u l=180n
M644 nw118 t201 0 0 nch w=1u l=180n
Cnw118 nw118 0 2f
CT205 t205 0 0.1f
M645 t205 nw116 0 0 nch w=1u l=180n
M646 t205 nw117 0 0 nch w=1u l=180n
M647 t205 nw118 0 0 nch w=1u l=180n
CT206 t206 0 0.1f
M648 t206 nw116 vdd vdd pch w=2u l=180n
CT207 t207 0 0.1f
M649 t207 nw117 t206 vdd pch w=2u l=180n
M650 t205 nw118 t207 vdd pch w=2u l=180n
M651 nw119 t205 vdd vdd pch w=2u l=180n
M652 nw119 t205 0 0 nch w=1u l=180n
Cnw119 nw119 0 2f
CT208 t208 0 0.1f
M653 t208 nw119 vdd vdd pch w=2u l=180n
M654 t208 nw119 0 0 nch w=1u l=180n
M655 nidx2 t208 vdd vdd pch w=2u l=180n
M656 nidx2 t208 0 0 nch w=1u l=180n
Cnidx2 nidx2 0 2f
CT209 t209 0 0.1f
M657 t209 nw50 0 0 nch w=1u l=180n
M658 t209 nw53 0 0 nch w=1u l=180n
M659 t209 nw56 0 0 nch w=1u l=180n
M660 t209 nw59 0 0 nch w=1u l=180n
CT210 t210 0 0.1f
M661 t210 nw50 vdd vdd pch w=2u l=180n
CT211 t211 0 0.1f
M662 t211 nw53 t210 vdd pch w=2u l=180n
CT212 t212 0 0.1f
M663 t212 nw56 t211 vdd pch w=2u l=180n
M664 t209 nw59 t212 vdd pch w=2u l=180n
M665 nw121 t209 vdd vdd pch w=2u l=180n
M666 nw121 t209 0 0 nch w=1u l=180n
Cnw121 nw121 0 2f
CT213 t213 0 0.1f
M667 t213 nw62 0 0 nch w=1u l=180n
M668 t213 nw65 0 0 nch w=1u l=180n
M669 t213 nw68 0 0 nch w=1u l=180n
M670 t213 nw71 0 0 nch w=1u l=180n
CT214 t214 0 0.1f
M671 t214 nw62 vdd vdd pch w=2u l=180n
CT215 t215 0 0.1f
M672 t215 nw65 t214 vdd pch w=2u l=180n
CT216 t216 0 0.1f
M673 t216 nw68 t215 vdd pch w=2u l=180n
M674 t213 nw71 t216 vdd pch w=2u l=180n
M675 nw122 t213 vdd vdd pch w=2u l=180n
M676 nw122 t213 0 0 nch w=1u l=180n
Cnw122 nw122 0 2f
CT217 t217 0 0.1f
M677 t217 nw98 0 0 nch w=1u l=180n
M678 t217 nw101 0 0 nch w=1u l=180n
M679 t217 nw104 0 0 nch w=1u l=180n
CT218 t218 0 0.1f
M680 t218 nw98 vdd vdd pch w=2u l=180n
CT219 t219 0 0.1f
M681 t219 nw101 t218 vdd pch w=2u l=180n
M682 t217 nw104 t219 vdd pch w=2u l=180n
M683 nw123 t217 vdd vdd pch w=2u l=180n
M684 nw123 t217 0 0 nch w=1u l=180n
Cnw123 nw123 0 2f
CT220 t220 0 0.1f
M685 t220 nw121 0 0 nch w=1u l=180n
M686 t220 nw122 0 0 nch w=1u l=180n
M687 t220 nw123 0 0 nch w=1u l=180n
CT221 t221 0 0.1f
M688 t221 nw121 vdd vdd pch w=2u l=180n
CT222 t222 0 0.1f
M689 t222 nw122 t221 vdd pch w=2u l=180n
M690 t220 nw123 t222 vdd pch w=2u l=180n
M691 nw124 t220 vdd vdd pch w=2u l=180n
M692 nw124 t220 0 0 nch w=1u l=180n
Cnw124 nw124 0 2f
CT223 t223 0 0.1f
M693 t223 nw124 vdd vdd pch w=2u l=180n
M694 t223 nw124 0 0 nch w=1u l=180n
M695 nidx3 t223 vdd vdd pch w=2u l=180n
M696 nidx3 t223 0 0 nch w=1u l=180n
Cnidx3 nidx3 0 2f
CT224 t224 0 0.1f
M697 t224 nw74 0 0 nch w=1u l=180n
M698 t224 nw77 0 0 nch w=1u l=180n
M699 t224 nw80 0 0 nch w=1u l=180n
M700 t224 nw83 0 0 nch w=1u l=180n
CT225 t225 0 0.1f
M701 t225 nw74 vdd vdd pch w=2u l=180n
CT226 t226 0 0.1f
M702 t226 nw77 t225 vdd pch w=2u l=180n
CT227 t227 0 0.1f
M703 t227 nw80 t226 vdd pch w=2u l=180n
M704 t224 nw83 t227 vdd pch w=2u l=180n
M705 nw126 t224 vdd vdd pch w=2u l=180n
M706 nw126 t224 0 0 nch w=1u l=180n
Cnw126 nw126 0 2f
CT228 t228 0 0.1f
M707 t228 nw86 0 0 nch w=1u l=180n
M708 t228 nw89 0 0 nch w=1u l=180n
M709 t228 nw92 0 0 nch w=1u l=180n
M710 t228 nw95 0 0 nch w=1u l=180n
CT229 t229 0 0.1f
M711 t229 nw86 vdd vdd pch w=2u l=180n
CT230 t230 0 0.1f
M712 t230 nw89 t229 vdd pch w=2u l=180n
CT231 t231 0 0.1f
M713 t231 nw92 t230 vdd pch w=2u l=180n
M714 t228 nw95 t231 vdd pch w=2u l=180n
M715 nw127 t228 vdd vdd pch w=2u l=180n
M716 nw127 t228 0 0 nch w=1u l=180n
Cnw127 nw127 0 2f
CT232 t232 0 0.1f
M717 t232 nw98 0 0 nch w=1u l=180n
M718 t232 nw101 0 0 nch w=1u l=180n
M719 t232 nw104 0 0 nch w=1u l=180n
CT233 t233 0 0.1f
M720 t233 nw98 vdd vdd pch w=2u l=180n
CT234 t234 0 0.1f
M721 t234 nw101 t233 vdd pch w=2u l=180n
M722 t232 nw104 t234 vdd pch w=2u l=180n
M723 nw128 t232 vdd vdd pch w=2u l=180n
M724 nw128 t232 0 0 nch w=1u l=180n
Cnw128 nw128 0 2f
CT235 t235 0 0.1f
M725 t235 nw126 0 0 nch w=1u l=180n
M726 t235 nw127 0 0 nch w=1u l=180n
M727 t235 nw128 0 0 nch w=1u l=180n
CT236 t236 0 0.1f
M728 t236 nw126 vdd vdd pch w=2u l=180n
CT237 t237 0 0.1f
M729 t237 nw127 t236 vdd pch w=2u l=180n
M730 t235 nw128 t237 vdd pch w=2u l=180n
M731 nw129 t235 vdd vdd pch w=2u l=180n
M732 nw129 t235 0 0 nch w=1u l=180n
Cnw129 nw129 0 2f
CT238 t238 0 0.1f
M733 t238 nw129 vdd vdd pch w=2u l=180n
M734 t238 nw129 0 0 nch w=1u l=180n
M735 nidx4 t238 vdd vdd pch w=2u l=180n
M736 nidx4 t238 0 0 nch w=1u l=180n
Cnidx4 nidx4 0 2f
CT239 t239 0 0.1f
M737 t239 nw105 vdd vdd pch w=2u l=180n
M738 t239 nw105 0 0 nch w=1u l=180n
M739 nany t239 vdd vdd pch w=2u l=180n
M740 nany t239 0 0 nch w=1u l=180n
Cnany nany 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: nidx0 nidx1 nidx2 nidx3 nidx4 nany
.end
