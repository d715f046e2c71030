* c6288 (c6288: 16 x 16 array multiplier): 1440 gates, 11872 transistors
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
VIN16 nb0 0 PULSE(0 1.8 3.2768e-05 20p 20p 6.5536e-05 0.000131072)
VIN17 nb1 0 PULSE(0 1.8 6.5536e-05 20p 20p 0.000131072 0.000262144)
VIN18 nb2 0 PULSE(0 1.8 0.000131072 20p 20p 0.000262144 0.000524288)
VIN19 nb3 0 PULSE(0 1.8 0.000262144 20p 20p 0.000524288 0.001048576)
VIN20 nb4 0 PULSE(0 1.8 0.000524288 20p 20p 0.001048576 0.002097152)
VIN21 nb5 0 PULSE(0 1.8 0.001048576 20p 20p 0.002097152 0.004194304)
VIN22 nb6 0 PULSE(0 1.8 0.002097152 20p 20p 0.004194304 0.008388608)
VIN23 nb7 0 PULSE(0 1.8 0.004194304 20p 20p 0.008388608 0.016777216)
VIN24 nb8 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN25 nb9 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN26 nb10 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN27 nb11 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN28 nb12 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN29 nb13 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN30 nb14 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN31 nb15 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
CT1 t1 0 0.1f
M1 t1 na0 vdd vdd pch w=2u l=180n
M2 t1 nb0 vdd vdd pch w=2u l=180n
CT2 t2 0 0.1f
M3 t1 na0 t2 0 nch w=1u l=180n
M4 t2 nb0 0 0 nch w=1u l=180n
M5 nw1 t1 vdd vdd pch w=2u l=180n
M6 nw1 t1 0 0 nch w=1u l=180n
Cnw1 nw1 0 2f
CT3 t3 0 0.1f
M7 t3 na1 vdd vdd pch w=2u l=180n
M8 t3 nb0 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M9 t3 na1 t4 0 nch w=1u l=180n
M10 t4 nb0 0 0 nch w=1u l=180n
M11 nw2 t3 vdd vdd pch w=2u l=180n
M12 nw2 t3 0 0 nch w=1u l=180n
Cnw2 nw2 0 2f
CT5 t5 0 0.1f
M13 t5 na2 vdd vdd pch w=2u l=180n
M14 t5 nb0 vdd vdd pch w=2u l=180n
CT6 t6 0 0.1f
M15 t5 na2 t6 0 nch w=1u l=180n
M16 t6 nb0 0 0 nch w=1u l=180n
M17 nw3 t5 vdd vdd pch w=2u l=180n
M18 nw3 t5 0 0 nch w=1u l=180n
Cnw3 nw3 0 2f
CT7 t7 0 0.1f
M19 t7 na3 vdd vdd pch w=2u l=180n
M20 t7 nb0 vdd vdd pch w=2u l=180n
CT8 t8 0 0.1f
M21 t7 na3 t8 0 nch w=1u l=180n
M22 t8 nb0 0 0 nch w=1u l=180n
M23 nw4 t7 vdd vdd pch w=2u l=180n
M24 nw4 t7 0 0 nch w=1u l=180n
Cnw4 nw4 0 2f
CT9 t9 0 0.1f
M25 t9 na4 vdd vdd pch w=2u l=180n
M26 t9 nb0 vdd vdd pch w=2u l=180n
CT10 t10 0 0.1f
M27 t9 na4 t10 0 nch w=1u l=180n
M28 t10 nb0 0 0 nch w=1u l=180n
M29 nw5 t9 vdd vdd pch w=2u l=180n
M30 nw5 t9 0 0 nch w=1u l=180n
Cnw5 nw5 0 2f
CT11 t11 0 0.1f
M31 t11 na5 vdd vdd pch w=2u l=180n
M32 t11 nb0 vdd vdd pch w=2u l=180n
CT12 t12 0 0.1f
M33 t11 na5 t12 0 nch w=1u l=180n
M34 t12 nb0 0 0 nch w=1u l=180n
M35 nw6 t11 vdd vdd pch w=2u l=180n
M36 nw6 t11 0 0 nch w=1u l=180n
Cnw6 nw6 0 2f
CT13 t13 0 0.1f
M37 t13 na6 vdd vdd pch w=2u l=180n
M38 t13 nb0 vdd vdd pch w=2u l=180n
CT14 t14 0 0.1f
M39 t13 na6 t14 0 nch w=1u l=180n
M40 t14 nb0 0 0 nch w=1u l=180n
M41 nw7 t13 vdd vdd pch w=2u l=180n
M42 nw7 t13 0 0 nch w=1u l=180n
Cnw7 nw7 0 2f
CT15 t15 0 0.1f
M43 t15 na7 vdd vdd pch w=2u l=180n
M44 t15 nb0 vdd vdd pch w=2u l=180n
CT16 t16 0 0.1f
M45 t15 na7 t16 0 nch w=1u l=180n
M46 t16 nb0 0 0 nch w=1u l=180n
M47 nw8 t15 vdd vdd pch w=2u l=180n
M48 nw8 t15 0 0 nch w=1u l=180n
Cnw8 nw8 0 2f
CT17 t17 0 0.1f
M49 t17 na8 vdd vdd pch w=2u l=180n
M50 t17 nb0 vdd vdd pch w=2u l=180n
CT18 t18 0 0.1f
M51 t17 na8 t18 0 nch w=1u l=180n
M52 t18 nb0 0 0 nch w=1u l=180n
M53 nw9 t17 vdd vdd pch w=2u l=180n
M54 nw9 t17 0 0 nch w=1u l=180n
Cnw9 nw9 0 2f
CT19 t19 0 0.1f
M55 t19 na9 vdd vdd pch w=2u l=180n
M56 t19 nb0 vdd vdd pch w=2u l=180n
CT20 t20 0 0.1f
M57 t19 na9 t20 0 nch w=1u l=180n
M58 t20 nb0 0 0 nch w=1u l=180n
M59 nw10 t19 vdd vdd pch w=2u l=180n
M60 nw10 t19 0 0 nch w=1u l=180n
Cnw10 nw10 0 2f
CT21 t21 0 0.1f
M61 t21 na10 vdd vdd pch w=2u l=180n
M62 t21 nb0 vdd vdd pch w=2u l=180n
CT22 t22 0 0.1f
M63 t21 na10 t22 0 nch w=1u l=180n
M64 t22 nb0 0 0 nch w=1u l=180n
M65 nw11 t21 vdd vdd pch w=2u l=180n
M66 nw11 t21 0 0 nch w=1u l=180n
Cnw11 nw11 0 2f
CT23 t23 0 0.1f
M67 t23 na11 vdd vdd pch w=2u l=180n
M68 t23 nb0 vdd vdd pch w=2u l=180n
CT24 t24 0 0.1f
M69 t23 na11 t24 0 nch w=1u l=180n
M70 t24 nb0 0 0 nch w=1u l=180n
M71 nw12 t23 vdd vdd pch w=2u l=180n
M72 nw12 t23 0 0 nch w=1u l=180n
Cnw12 nw12 0 2f
CT25 t25 0 0.1f
M73 t25 na12 vdd vdd pch w=2u l=180n
M74 t25 nb0 vdd vdd pch w=2u l=180n
CT26 t26 0 0.1f
M75 t25 na12 t26 0 nch w=1u l=180n
M76 t26 nb0 0 0 nch w=1u l=180n
M77 nw13 t25 vdd vdd pch w=2u l=180n
M78 nw13 t25 0 0 nch w=1u l=180n
Cnw13 nw13 0 2f
CT27 t27 0 0.1f
M79 t27 na13 vdd vdd pch w=2u l=180n
M80 t27 nb0 vdd vdd pch w=2u l=180n
CT28 t28 0 0.1f
M81 t27 na13 t28 0 nch w=1u l=180n
M82 t28 nb0 0 0 nch w=1u l=180n
M83 nw14 t27 vdd vdd pch w=2u l=180n
M84 nw14 t27 0 0 nch w=1u l=180n
Cnw14 nw14 0 2f
CT29 t29 0 0.1f
M85 t29 na14 vdd vdd pch w=2u l=180n
M86 t29 nb0 vdd vdd pch w=2u l=180n
CT30 t30 0 0.1f
M87 t29 na14 t30 0 nch w=1u l=180n
M88 t30 nb0 0 0 nch w=1u l=180n
M89 nw15 t29 vdd vdd pch w=2u l=180n
M90 nw15 t29 0 0 nch w=1u l=180n
Cnw15 nw15 0 2f
CT31 t31 0 0.1f
M91 t31 na15 vdd vdd pch w=2u l=180n
M92 t31 nb0 vdd vdd pch w=2u l=180n
CT32 t32 0 0.1f
M93 t31 na15 t32 0 nch w=1u l=180n
M94 t32 nb0 0 0 nch w=1u l=180n
M95 nw16 t31 vdd vdd pch w=2u l=180n
M96 nw16 t31 0 0 nch w=1u l=180n
Cnw16 nw16 0 2f
CT33 t33 0 0.1f
M97 t33 na0 vdd vdd pch w=2u l=180n
M98 t33 nb1 vdd vdd pch w=2u l=180n
CT34 t34 0 0.1f
M99 t33 na0 t34 0 nch w=1u l=180n
M100 t34 nb1 0 0 nch w=1u l=180n
M101 nw17 t33 vdd vdd pch w=2u l=180n
M102 nw17 t33 0 0 nch w=1u l=180n
Cnw17 nw17 0 2f
CT35 t35 0 0.1f
M103 t35 na1 vdd vdd pch w=2u l=180n
M104 t35 nb1 vdd vdd pch w=2u l=180n
CT36 t36 0 0.1f
M105 t35 na1 t36 0 nch w=1u l=180n
M106 t36 nb1 0 0 nch w=1u l=180n
M107 nw18 t35 vdd vdd pch w=2u l=180n
M108 nw18 t35 0 0 nch w=1u l=180n
Cnw18 nw18 0 2f
CT37 t37 0 0.1f
M109 t37 na2 vdd vdd pch w=2u l=180n
M110 t37 nb1 vdd vdd pch w=2u l=180n
CT38 t38 0 0.1f
M111 t37 na2 t38 0 nch w=1u l=180n
M112 t38 nb1 0 0 nch w=1u l=180n
M113 nw19 t37 vdd vdd pch w=2u l=180n
M114 nw19 t37 0 0 nch w=1u l=180n
Cnw19 nw19 0 2f
CT39 t39 0 0.1f
M115 t39 na3 vdd vdd pch w=2u l=180n
M116 t39 nb1 vdd vdd pch w=2u l=180n
CT40 t40 0 0.1f
M117 t39 na3 t40 0 nch w=1u l=180n
M118 t40 nb1 0 0 nch w=1u l=180n
M119 nw20 t39 vdd vdd pch w=2u l=180n
M120 nw20 t39 0 0 nch w=1u l=180n
Cnw20 nw20 0 2f
CT41 t41 0 0.1f
M121 t41 na4 vdd vdd pch w=2u l=180n
M122 t41 nb1 vdd vdd pch w=2u l=180n
CT42 t42 0 0.1f
M123 t41 na4 t42 0 nch w=1u l=180n
M124 t42 nb1 0 0 nch w=1u l=180n
M125 nw21 t41 vdd vdd pch w=2u l=180n
M126 nw21 t41 0 0 nch w=1u l=180n
Cnw21 nw21 0 2f
CT43 t43 0 0.1f
M127 t43 na5 vdd vdd pch w=2u l=180n
M128 t43 nb1 vdd vdd pch w=2u l=180n
CT44 t44 0 0.1f
M129 t43 na5 t44 0 nch w=1u l=180n
M130 t44 nb1 0 0 nch w=1u l=180n
M131 nw22 t43 vdd vdd pch w=2u l=180n
M132 nw22 t43 0 0 nch w=1u l=180n
Cnw22 nw22 0 2f
CT45 t45 0 0.1f
M133 t45 na6 vdd vdd pch w=2u l=180n
M134 t45 nb1 vdd vdd pch w=2u l=180n
CT46 t46 0 0.1f
M135 t45 na6 t46 0 nch w=1u l=180n
M136 t46 nb1 0 0 nch w=1u l=180n
M137 nw23 t45 vdd vdd pch w=2u l=180n
M138 nw23 t45 0 0 nch w=1u l=180n
Cnw23 nw23 0 2f
CT47 t47 0 0.1f
M139 t47 na7 vdd vdd pch w=2u l=180n
M140 t47 nb1 vdd vdd pch w=2u l=180n
CT48 t48 0 0.1f
M141 t47 na7 t48 0 nch w=1u l=180n
M142 t48 nb1 0 0 nch w=1u l=180n
M143 nw24 t47 vdd vdd pch w=2u l=180n
M144 nw24 t47 0 0 nch w=1u l=180n
Cnw24 nw24 0 2f
CT49 t49 0 0.1f
M145 t49 na8 vdd vdd pch w=2u l=180n
M146 t49 nb1 vdd vdd pch w=2u l=180n
CT50 t50 0 0.1f
M147 t49 na8 t50 0 nch w=1u l=180n
M148 t50 nb1 0 0 nch w=1u l=180n
M149 nw25 t49 vdd vdd pch w=2u l=180n
M150 nw25 t49 0 0 nch w=1u l=180n
Cnw25 nw25 0 2f
CT51 t51 0 0.1f
M151 t51 na9 vdd vdd pch w=2u l=180n
M152 t51 nb1 vdd vdd pch w=2u l=180n
CT52 t52 0 0.1f
M153 t51 na9 t52 0 nch w=1u l=180n
M154 t52 nb1 0 0 nch w=1u l=180n
M155 nw26 t51 vdd vdd pch w=2u l=180n
M156 nw26 t51 0 0 nch w=1u l=180n
Cnw26 nw26 0 2f
CT53 t53 0 0.1f
M157 t53 na10 vdd vdd pch w=2u l=180n
M158 t53 nb1 vdd vdd pch w=2u l=180n
CT54 t54 0 0.1f
M159 t53 na10 t54 0 nch w=1u l=180n
M160 t54 nb1 0 0 nch w=1u l=180n
M161 nw27 t53 vdd vdd pch w=2u l=180n
M162 nw27 t53 0 0 nch w=1u l=180n
Cnw27 nw27 0 2f
CT55 t55 0 0.1f
M163 t55 na11 vdd vdd pch w=2u l=180n
M164 t55 nb1 vdd vdd pch w=2u l=180n
CT56 t56 0 0.1f
M165 t55 na11 t56 0 nch w=1u l=180n
M166 t56 nb1 0 0 nch w=1u l=180n
M167 nw28 t55 vdd vdd pch w=2u l=180n
M168 nw28 t55 0 0 nch w=1u l=180n
Cnw28 nw28 0 2f
CT57 t57 0 0.1f
M169 t57 na12 vdd vdd pch w=2u l=180n
M170 t57 nb1 vdd vdd pch w=2u l=180n
CT58 t58 0 0.1f
M171 t57 na12 t58 0 nch w=1u l=180n
M172 t58 nb1 0 0 nch w=1u l=180n
M173 nw29 t57 vdd vdd pch w=2u l=180n
M174 nw29 t57 0 0 nch w=1u l=180n
Cnw29 nw29 0 2f
CT59 t59 0 0.1f
M175 t59 na13 vdd vdd pch w=2u l=180n
M176 t59 nb1 vdd vdd pch w=2u l=180n
CT60 t60 0 0.1f
M177 t59 na13 t60 0 nch w=1u l=180n
M178 t60 nb1 0 0 nch w=1u l=180n
M179 nw30 t59 vdd vdd pch w=2u l=180n
M180 nw30 t59 0 0 nch w=1u l=180n
Cnw30 nw30 0 2f
CT61 t61 0 0.1f
M181 t61 na14 vdd vdd pch w=2u l=180n
M182 t61 nb1 vdd vdd pch w=2u l=180n
CT62 t62 0 0.1f
M183 t61 na14 t62 0 nch w=1u l=180n
M184 t62 nb1 0 0 nch w=1u l=180n
M185 nw31 t61 vdd vdd pch w=2u l=180n
M186 nw31 t61 0 0 nch w=1u l=180n
Cnw31 nw31 0 2f
CT63 t63 0 0.1f
M187 t63 na15 vdd vdd pch w=2u l=180n
M188 t63 nb1 vdd vdd pch w=2u l=180n
CT64 t64 0 0.1f
M189 t63 na15 t64 0 nch w=1u l=180n
M190 t64 nb1 0 0 nch w=1u l=180n
M191 nw32 t63 vdd vdd pch w=2u l=180n
M192 nw32 t63 0 0 nch w=1u l=180n
Cnw32 nw32 0 2f
CT65 t65 0 0.1f
M193 t65 na0 vdd vdd pch w=2u l=180n
M194 t65 nb2 vdd vdd pch w=2u l=180n
CT66 t66 0 0.1f
M195 t65 na0 t66 0 nch w=1u l=180n
M196 t66 nb2 0 0 nch w=1u l=180n
M197 nw33 t65 vdd vdd pch w=2u l=180n
M198 nw33 t65 0 0 nch w=1u l=180n
Cnw33 nw33 0 2f
CT67 t67 0 0.1f
M199 t67 na1 vdd vdd pch w=2u l=180n
M200 t67 nb2 vdd vdd pch w=2u l=180n
CT68 t68 0 0.1f
M201 t67 na1 t68 0 nch w=1u l=180n
M202 t68 nb2 0 0 nch w=1u l=180n
M203 nw34 t67 vdd vdd pch w=2u l=180n
M204 nw34 t67 0 0 nch w=1u l=180n
Cnw34 nw34 0 2f
CT69 t69 0 0.1f
M205 t69 na2 vdd vdd pch w=2u l=180n
M206 t69 nb2 vdd vdd pch w=2u l=180n
CT70 t70 0 0.1f
M207 t69 na2 t70 0 nch w=1u l=180n
M208 t70 nb2 0 0 nch w=1u l=180n
M209 nw35 t69 vdd vdd pch w=2u l=180n
M210 nw35 t69 0 0 nch w=1u l=180n
Cnw35 nw35 0 2f
CT71 t71 0 0.1f
M211 t71 na3 vdd vdd pch w=2u l=180n
M212 t71 nb2 vdd vdd pch w=2u l=180n
CT72 t72 0 0.1f
M213 t71 na3 t72 0 nch w=1u l=180n
M214 t72 nb2 0 0 nch w=1u l=180n
M215 nw36 t71 vdd vdd pch w=2u l=180n
M216 nw36 t71 0 0 nch w=1u l=180n
Cnw36 nw36 0 2f
CT73 t73 0 0.1f
M217 t73 na4 vdd vdd pch w=2u l=180n
M218 t73 nb2 vdd vdd pch w=2u l=180n
CT74 t74 0 0.1f
M219 t73 na4 t74 0 nch w=1u l=180n
M220 t74 nb2 0 0 nch w=1u l=180n
M221 nw37 t73 vdd vdd pch w=2u l=180n
M222 nw37 t73 0 0 nch w=1u l=180n
Cnw37 nw37 0 2f
CT75 t75 0 0.1f
M223 t75 na5 vdd vdd pch w=2u l=180n
M224 t75 nb2 vdd vdd pch w=2u l=180n
CT76 t76 0 0.1f
M225 t75 na5 t76 0 nch w=1u l=180n
M226 t76 nb2 0 0 nch w=1u l=180n
M227 nw38 t75 vdd vdd pch w=2u l=180n
M228 nw38 t75 0 0 nch w=1u l=180n
Cnw38 nw38 0 2f
CT77 t77 0 0.1f
M229 t77 na6 vdd vdd pch w=2u l=180n
M230 t77 nb2 vdd vdd pch w=2u l=180n
CT78 t78 0 0.1f
M231 t77 na6 t78 0 nch w=1u l=180n
M232 t78 nb2 0 0 nch w=1u l=180n
M233 nw39 t77 vdd vdd pch w=2u l=180n
M234 nw39 t77 0 0 nch w=1u l=180n
Cnw39 nw39 0 2f
CT79 t79 0 0.1f
M235 t79 na7 vdd vdd pch w=2u l=180n
M236 t79 nb2 vdd vdd pch w=2u l=180n
CT80 t80 0 0.1f
M237 t79 na7 t80 0 nch w=1u l=180n
M238 t80 nb2 0 0 nch w=1u l=180n
M239 nw40 t79 vdd vdd pch w=2u l=180n
M240 nw40 t79 0 0 nch w=1u l=180n
Cnw40 nw40 0 2f
CT81 t81 0 0.1f
M241 t81 na8 vdd vdd pch w=2u l=180n
M242 t81 nb2 vdd vdd pch w=2u l=180n
CT82 t82 0 0.1f
M243 t81 na8 t82 0 nch w=1u l=180n
M244 t82 nb2 0 0 nch w=1u l=180n
M245 nw41 t81 vdd vdd pch w=2u l=180n
M246 nw41 t81 0 0 nch w=1u l=180n
Cnw41 nw41 0 2f
CT83 t83 0 0.1f
M247 t83 na9 vdd vdd pch w=2u l=180n
M248 t83 nb2 vdd vdd pch w=2u l=180n
CT84 t84 0 0.1f
M249 t83 na9 t84 0 nch w=1u l=180n
M250 t84 nb2 0 0 nch w=1u l=180n
M251 nw42 t83 vdd vdd pch w=2u l=180n
M252 nw42 t83 0 0 nch w=1u l=180n
Cnw42 nw42 0 2f
CT85 t85 0 0.1f
M253 t85 na10 vdd vdd pch w=2u l=180n
M254 t85 nb2 vdd vdd pch w=2u l=180n
CT86 t86 0 0.1f
M255 t85 na10 t86 0 nch w=1u l=180n
M256 t86 nb2 0 0 nch w=1u l=180n
M257 nw43 t85 vdd vdd pch w=2u l=180n
M258 nw43 t85 0 0 nch w=1u l=180n
Cnw43 nw43 0 2f
CT87 t87 0 0.1f
M259 t87 na11 vdd vdd pch w=2u l=180n
M260 t87 nb2 vdd vdd pch w=2u l=180n
CT88 t88 0 0.1f
M261 t87 na11 t88 0 nch w=1u l=180n
M262 t88 nb2 0 0 nch w=1u l=180n
M263 nw44 t87 vdd vdd pch w=2u l=180n
M264 nw44 t87 0 0 nch w=1u l=180n
Cnw44 nw44 0 2f
CT89 t89 0 0.1f
M265 t89 na12 vdd vdd pch w=2u l=180n
M266 t89 nb2 vdd vdd pch w=2u l=180n
CT90 t90 0 0.1f
M267 t89 na12 t90 0 nch w=1u l=180n
M268 t90 nb2 0 0 nch w=1u l=180n
M269 nw45 t89 vdd vdd pch w=2u l=180n
M270 nw45 t89 0 0 nch w=1u l=180n
Cnw45 nw45 0 2f
CT91 t91 0 0.1f
M271 t91 na13 vdd vdd pch w=2u l=180n
M272 t91 nb2 vdd vdd pch w=2u l=180n
CT92 t92 0 0.1f
M273 t91 na13 t92 0 nch w=1u l=180n
M274 t92 nb2 0 0 nch w=1u l=180n
M275 nw46 t91 vdd vdd pch w=2u l=180n
M276 nw46 t91 0 0 nch w=1u l=180n
Cnw46 nw46 0 2f
CT93 t93 0 0.1f
M277 t93 na14 vdd vdd pch w=2u l=180n
M278 t93 nb2 vdd vdd pch w=2u l=180n
CT94 t94 0 0.1f
M279 t93 na14 t94 0 nch w=1u l=180n
M280 t94 nb2 0 0 nch w=1u l=180n
M281 nw47 t93 vdd vdd pch w=2u l=180n
M282 nw47 t93 0 0 nch w=1u l=180n
Cnw47 nw47 0 2f
CT95 t95 0 0.1f
M283 t95 na15 vdd vdd pch w=2u l=180n
M284 t95 nb2 vdd vdd pch w=2u l=180n
CT96 t96 0 0.1f
M285 t95 na15 t96 0 nch w=1u l=180n
M286 t96 nb2 0 0 nch w=1u l=180n
M287 nw48 t95 vdd vdd pch w=2u l=180n
M288 nw48 t95 0 0 nch w=1u l=180n
Cnw48 nw48 0 2f
CT97 t97 0 0.1f
M289 t97 na0 vdd vdd pch w=2u l=180n
M290 t97 nb3 vdd vdd pch w=2u l=180n
CT98 t98 0 0.1f
M291 t97 na0 t98 0 nch w=1u l=180n
M292 t98 nb3 0 0 nch w=1u l=180n
M293 nw49 t97 vdd vdd pch w=2u l=180n
M294 nw49 t97 0 0 nch w=1u l=180n
Cnw49 nw49 0 2f
CT99 t99 0 0.1f
M295 t99 na1 vdd vdd pch w=2u l=180n
M296 t99 nb3 vdd vdd pch w=2u l=180n
CT100 t100 0 0.1f
M297 t99 na1 t100 0 nch w=1u l=180n
M298 t100 nb3 0 0 nch w=1u l=180n
M299 nw50 t99 vdd vdd pch w=2u l=180n
M300 nw50 t99 0 0 nch w=1u l=180n
Cnw50 nw50 0 2f
CT101 t101 0 0.1f
M301 t101 na2 vdd vdd pch w=2u l=180n
M302 t101 nb3 vdd vdd pch w=2u l=180n
CT102 t102 0 0.1f
M303 t101 na2 t102 0 nch w=1u l=180n
M304 t102 nb3 0 0 nch w=1u l=180n
M305 nw51 t101 vdd vdd pch w=2u l=180n
M306 nw51 t101 0 0 nch w=1u l=180n
Cnw51 nw51 0 2f
CT103 t103 0 0.1f
M307 t103 na3 vdd vdd pch w=2u l=180n
M308 t103 nb3 vdd vdd pch w=2u l=180n
CT104 t104 0 0.1f
M309 t103 na3 t104 0 nch w=1u l=180n
M310 t104 nb3 0 0 nch w=1u l=180n
M311 nw52 t103 vdd vdd pch w=2u l=180n
M312 nw52 t103 0 0 nch w=1u l=180n
Cnw52 nw52 0 2f
CT105 t105 0 0.1f
M313 t105 na4 vdd vdd pch w=2u l=180n
M314 t105 nb3 vdd vdd pch w=2u l=180n
CT106 t106 0 0.1f
M315 t105 na4 t106 0 nch w=1u l=180n
M316 t106 nb3 0 0 nch w=1u l=180n
M317 nw53 t105 vdd vdd pch w=2u l=180n
M318 nw53 t105 0 0 nch w=1u l=180n
Cnw53 nw53 0 2f
CT107 t107 0 0.1f
M319 t107 na5 vdd vdd pch w=2u l=180n
M320 t107 nb3 vdd vdd pch w=2u l=180n
CT108 t108 0 0.1f
M321 t107 na5 t108 0 nch w=1u l=180n
M322 t108 nb3 0 0 nch w=1u l=180n
M323 nw54 t107 vdd vdd pch w=2u l=180n
M324 nw54 t107 0 0 nch w=1u l=180n
Cnw54 nw54 0 2f
CT109 t109 0 0.1f
M325 t109 na6 vdd vdd pch w=2u l=180n
M326 t109 nb3 vdd vdd pch w=2u l=180n
CT110 t110 0 0.1f
M327 t109 na6 t110 0 nch w=1u l=180n
M328 t110 nb3 0 0 nch w=1u l=180n
M329 nw55 t109 vdd vdd pch w=2u l=180n
M330 nw55 t109 0 0 nch w=1u l=180n
Cnw55 nw55 0 2f
CT111 t111 0 0.1f
M331 t111 na7 vdd vdd pch w=2u l=180n
M332 t111 nb3 vdd vdd pch w=2u l=180n
CT112 t112 0 0.1f
M333 t111 na7 t112 0 nch w=1u l=180n
M334 t112 nb3 0 0 nch w=1u l=180n
M335 nw56 t111 vdd vdd pch w=2u l=180n
M336 nw56 t111 0 0 nch w=1u l=180n
Cnw56 nw56 0 2f
CT113 t113 0 0.1f
M337 t113 na8 vdd vdd pch w=2u l=180n
M338 t113 nb3 vdd vdd pch w=2u l=180n
CT114 t114 0 0.1f
M339 t113 na8 t114 0 nch w=1u l=180n
M340 t114 nb3 0 0 nch w=1u l=180n
M341 nw57 t113 vdd vdd pch w=2u l=180n
M342 nw57 t113 0 0 nch w=1u l=180n
Cnw57 nw57 0 2f
CT115 t115 0 0.1f
M343 t115 na9 vdd vdd pch w=2u l=180n
M344 t115 nb3 vdd vdd pch w=2u l=180n
CT116 t116 0 0.1f
M345 t115 na9 t116 0 nch w=1u l=180n
M346 t116 nb3 0 0 nch w=1u l=180n
M347 nw58 t115 vdd vdd pch w=2u l=180n
M348 nw58 t115 0 0 nch w=1u l=180n
Cnw58 nw58 0 2f
CT117 t117 0 0.1f
M349 t117 na10 vdd vdd pch w=2u l=180n
M350 t117 nb3 vdd vdd pch w=2u l=180n
CT118 t118 0 0.1f
M351 t117 na10 t118 0 nch w=1u l=180n
M352 t118 nb3 0 0 nch w=1u l=180n
M353 nw59 t117 vdd vdd pch w=2u l=180n
M354 nw59 t117 0 0 nch w=1u l=180n
Cnw59 nw59 0 2f
CT119 t119 0 0.1f
M355 t119 na11 vdd vdd pch w=2u l=180n
M356 t119 nb3 vdd vdd pch w=2u l=180n
CT120 t120 0 0.1f
M357 t119 na11 t120 0 nch w=1u l=180n
M358 t120 nb3 0 0 nch w=1u l=180n
M359 nw60 t119 vdd vdd pch w=2u l=180n
M360 nw60 t119 0 0 nch w=1u l=180n
Cnw60 nw60 0 2f
CT121 t121 0 0.1f
M361 t121 na12 vdd vdd pch w=2u l=180n
M362 t121 nb3 vdd vdd pch w=2u l=180n
CT122 t122 0 0.1f
M363 t121 na12 t122 0 nch w=1u l=180n
M364 t122 nb3 0 0 nch w=1u l=180n
M365 nw61 t121 vdd vdd pch w=2u l=180n
M366 nw61 t121 0 0 nch w=1u l=180n
Cnw61 nw61 0 2f
CT123 t123 0 0.1f
M367 t123 na13 vdd vdd pch w=2u l=180n
M368 t123 nb3 vdd vdd pch w=2u l=180n
CT124 t124 0 0.1f
M369 t123 na13 t124 0 nch w=1u l=180n
M370 t124 nb3 0 0 nch w=1u l=180n
M371 nw62 t123 vdd vdd pch w=2u l=180n
M372 nw62 t123 0 0 nch w=1u l=180n
Cnw62 nw62 0 2f
CT125 t125 0 0.1f
M373 t125 na14 vdd vdd pch w=2u l=180n
M374 t125 nb3 vdd vdd pch w=2u l=180n
CT126 t126 0 0.1f
M375 t125 na14 t126 0 nch w=1u l=180n
M376 t126 nb3 0 0 nch w=1u l=180n
M377 nw63 t125 vdd vdd pch w=2u l=180n
M378 nw63 t125 0 0 nch w=1u l=180n
Cnw63 nw63 0 2f
CT127 t127 0 0.1f
M379 t127 na15 vdd vdd pch w=2u l=180n
M380 t127 nb3 vdd vdd pch w=2u l=180n
CT128 t128 0 0.1f
M381 t127 na15 t128 0 nch w=1u l=180n
M382 t128 nb3 0 0 nch w=1u l=180n
M383 nw64 t127 vdd vdd pch w=2u l=180n
M384 nw64 t127 0 0 nch w=1u l=180n
Cnw64 nw64 0 2f
CT129 t129 0 0.1f
M385 t129 na0 vdd vdd pch w=2u l=180n
M386 t129 nb4 vdd vdd pch w=2u l=180n
CT130 t130 0 0.1f
M387 t129 na0 t130 0 nch w=1u l=180n
M388 t130 nb4 0 0 nch w=1u l=180n
M389 nw65 t129 vdd vdd pch w=2u l=180n
M390 nw65 t129 0 0 nch w=1u l=180n
Cnw65 nw65 0 2f
CT131 t131 0 0.1f
M391 t131 na1 vdd vdd pch w=2u l=180n
M392 t131 nb4 vdd vdd pch w=2u l=180n
CT132 t132 0 0.1f
M393 t131 na1 t132 0 nch w=1u l=180n
M394 t132 nb4 0 0 nch w=1u l=180n
M395 nw66 t131 vdd vdd pch w=2u l=180n
M396 nw66 t131 0 0 nch w=1u l=180n
Cnw66 nw66 0 2f
CT133 t133 0 0.1f
M397 t133 na2 vdd vdd pch w=2u l=180n
M398 t133 nb4 vdd vdd pch w=2u l=180n
CT134 t134 0 0.1f
M399 t133 na2 t134 0 nch w=1u l=180n
M400 t134 nb4 0 0 nch w=1u l=180n
M401 nw67 t133 vdd vdd pch w=2u l=180n
M402 nw67 t133 0 0 nch w=1u l=180n
Cnw67 nw67 0 2f
CT135 t135 0 0.1f
M403 t135 na3 vdd vdd pch w=2u l=180n
M404 t135 nb4 vdd vdd pch w=2u l=180n
CT136 t136 0 0.1f
M405 t135 na3 t136 0 nch w=1u l=180n
M406 t136 nb4 0 0 nch w=1u l=180n
M407 nw68 t135 vdd vdd pch w=2u l=180n
M408 nw68 t135 0 0 nch w=1u l=180n
Cnw68 nw68 0 2f
CT137 t137 0 0.1f
M409 t137 na4 vdd vdd pch w=2u l=180n
M410 t137 nb4 vdd vdd pch w=2u l=180n
CT138 t138 0 0.1f
M411 t137 na4 t138 0 nch w=1u l=180n
M412 t138 nb4 0 0 nch w=1u l=180n
M413 nw69 t137 vdd vdd pch w=2u l=180n
M414 nw69 t137 0 0 nch w=1u l=180n
Cnw69 nw69 0 2f
CT139 t139 0 0.1f
M415 t139 na5 vdd vdd pch w=2u l=180n
M416 t139 nb4 vdd vdd pch w=2u l=180n
CT140 t140 0 0.1f
M417 t139 na5 t140 0 nch w=1u l=180n
M418 t140 nb4 0 0 nch w=1u l=180n
M419 nw70 t139 vdd vdd pch w=2u l=180n
M420 nw70 t139 0 0 nch w=1u l=180n
Cnw70 nw70 0 2f
CT141 t141 0 0.1f
M421 t141 na6 vdd vdd pch w=2u l=180n
M422 t141 nb4 vdd vdd pch w=2u l=180n
CT142 t142 0 0.1f
M423 t141 na6 t142 0 nch w=1u l=180n
M424 t142 nb4 0 0 nch w=1u l=180n
M425 nw71 t141 vdd vdd pch w=2u l=180n
M426 nw71 t141 0 0 nch w=1u l=180n
Cnw71 nw71 0 2f
CT143 t143 0 0.1f
M427 t143 na7 vdd vdd pch w=2u l=180n
M428 t143 nb4 vdd vdd pch w=2u l=180n
CT144 t144 0 0.1f
M429 t143 na7 t144 0 nch w=1u l=180n
M430 t144 nb4 0 0 nch w=1u l=180n
M431 nw72 t143 vdd vdd pch w=2u l=180n
M432 nw72 t143 0 0 nch w=1u l=180n
Cnw72 nw72 0 2f
CT145 t145 0 0.1f
M433 t145 na8 vdd vdd pch w=2u l=180n
M434 t145 nb4 vdd vdd pch w=2u l=180n
CT146 t146 0 0.1f
M435 t145 na8 t146 0 nch w=1u l=180n
M436 t146 nb4 0 0 nch w=1u l=180n
M437 nw73 t145 vdd vdd pch w=2u l=180n
M438 nw73 t145 0 0 nch w=1u l=180n
Cnw73 nw73 0 2f
CT147 t147 0 0.1f
M439 t147 na9 vdd vdd pch w=2u l=180n
M440 t147 nb4 vdd vdd pch w=2u l=180n
CT148 t148 0 0.1f
M441 t147 na9 t148 0 nch w=1u l=180n
M442 t148 nb4 0 0 nch w=1u l=180n
M443 nw74 t147 vdd vdd pch w=2u l=180n
M444 nw74 t147 0 0 nch w=1u l=180n
Cnw74 nw74 0 2f
CT149 t149 0 0.1f
M445 t149 na10 vdd vdd pch w=2u l=180n
M446 t149 nb4 vdd vdd pch w=2u l=180n
CT150 t150 0 0.1f
M447 t149 na10 t150 0 nch w=1u l=180n
M448 t150 nb4 0 0 nch w=1u l=180n
M449 nw75 t149 vdd vdd pch w=2u l=180n
M450 nw75 t149 0 0 nch w=1u l=180n
Cnw75 nw75 0 2f
CT151 t151 0 0.1f
M451 t151 na11 vdd vdd pch w=2u l=180n
M452 t151 nb4 vdd vdd pch w=2u l=180n
CT152 t152 0 0.1f
M453 t151 na11 t152 0 nch w=1u l=180n
M454 t152 nb4 0 0 nch w=1u l=180n
M455 nw76 t151 vdd vdd pch w=2u l=180n
M456 nw76 t151 0 0 nch w=1u l=180n
Cnw76 nw76 0 2f
CT153 t153 0 0.1f
M457 t153 na12 vdd vdd pch w=2u l=180n
M458 t153 nb4 vdd vdd pch w=2u l=180n
CT154 t154 0 0.1f
M459 t153 na12 t154 0 nch w=1u l=180n
M460 t154 nb4 0 0 nch w=1u l=180n
M461 nw77 t153 vdd vdd pch w=2u l=180n
M462 nw77 t153 0 0 nch w=1u l=180n
Cnw77 nw77 0 2f
CT155 t155 0 0.1f
M463 t155 na13 vdd vdd pch w=2u l=180n
M464 t155 nb4 vdd vdd pch w=2u l=180n
CT156 t156 0 0.1f
M465 t155 na13 t156 0 nch w=1u l=180n
M466 t156 nb4 0 0 nch w=1u l=180n
M467 nw78 t155 vdd vdd pch w=2u l=180n
M468 nw78 t155 0 0 nch w=1u l=180n
Cnw78 nw78 0 2f
CT157 t157 0 0.1f
M469 t157 na14 vdd vdd pch w=2u l=180n
M470 t157 nb4 vdd vdd pch w=2u l=180n
CT158 t158 0 0.1f
M471 t157 na14 t158 0 nch w=1u l=180n
M472 t158 nb4 0 0 nch w=1u l=180n
M473 nw79 t157 vdd vdd pch w=2u l=180n
M474 nw79 t157 0 0 nch w=1u l=180n
Cnw79 nw79 0 2f
CT159 t159 0 0.1f
M475 t159 na15 vdd vdd pch w=2u l=180n
M476 t159 nb4 vdd vdd pch w=2u l=180n
CT160 t160 0 0.1f
M477 t159 na15 t160 0 nch w=1u l=180n
M478 t160 nb4 0 0 nch w=1u l=180n
M479 nw80 t159 vdd vdd pch w=2u l=180n
M480 nw80 t159 0 0 nch w=1u l=180n
Cnw80 nw80 0 2f
CT161 t161 0 0.1f
M481 t161 na0 vdd vdd pch w=2u l=180n
M482 t161 nb5 vdd vdd pch w=2u l=180n
CT162 t162 0 0.1f
M483 t161 na0 t162 0 nch w=1u l=180n
M484 t162 nb5 0 0 nch w=1u l=180n
M485 nw81 t161 vdd vdd pch w=2u l=180n
M486 nw81 t161 0 0 nch w=1u l=180n
Cnw81 nw81 0 2f
CT163 t163 0 0.1f
M487 t163 na1 vdd vdd pch w=2u l=180n
M488 t163 nb5 vdd vdd pch w=2u l=180n
CT164 t164 0 0.1f
M489 t163 na1 t164 0 nch w=1u l=180n
M490 t164 nb5 0 0 nch w=1u l=180n
M491 nw82 t163 vdd vdd pch w=2u l=180n
M492 nw82 t163 0 0 nch w=1u l=180n
Cnw82 nw82 0 2f
CT165 t165 0 0.1f
M493 t165 na2 vdd vdd pch w=2u l=180n
M494 t165 nb5 vdd vdd pch w=2u l=180n
CT166 t166 0 0.1f
M495 t165 na2 t166 0 nch w=1u l=180n
M496 t166 nb5 0 0 nch w=1u l=180n
M497 nw83 t165 vdd vdd pch w=2u l=180n
M498 nw83 t165 0 0 nch w=1u l=180n
Cnw83 nw83 0 2f
CT167 t167 0 0.1f
M499 t167 na3 vdd vdd pch w=2u l=180n
M500 t167 nb5 vdd vdd pch w=2u l=180n
CT168 t168 0 0.1f
M501 t167 na3 t168 0 nch w=1u l=180n
M502 t168 nb5 0 0 nch w=1u l=180n
M503 nw84 t167 vdd vdd pch w=2u l=180n
M504 nw84 t167 0 0 nch w=1u l=180n
Cnw84 nw84 0 2f
CT169 t169 0 0.1f
M505 t169 na4 vdd vdd pch w=2u l=180n
M506 t169 nb5 vdd vdd pch w=2u l=180n
CT170 t170 0 0.1f
M507 t169 na4 t170 0 nch w=1u l=180n
M508 t170 nb5 0 0 nch w=1u l=180n
M509 nw85 t169 vdd vdd pch w=2u l=180n
M510 nw85 t169 0 0 nch w=1u l=180n
Cnw85 nw85 0 2f
CT171 t171 0 0.1f
M511 t171 na5 vdd vdd pch w=2u l=180n
M512 t171 nb5 vdd vdd pch w=2u l=180n
CT172 t172 0 0.1f
M513 t171 na5 t172 0 nch w=1u l=180n
M514 t172 nb5 0 0 nch w=1u l=180n
M515 nw86 t171 vdd vdd pch w=2u l=180n
M516 nw86 t171 0 0 nch w=1u l=180n
Cnw86 nw86 0 2f
CT173 t173 0 0.1f
M517 t173 na6 vdd vdd pch w=2u l=180n
M518 t173 nb5 vdd vdd pch w=2u l=180n
CT174 t174 0 0.1f
M519 t173 na6 t174 0 nch w=1u l=180n
M520 t174 nb5 0 0 nch w=1u l=180n
M521 nw87 t173 vdd vdd pch w=2u l=180n
M522 nw87 t173 0 0 nch w=1u l=180n
Cnw87 nw87 0 2f
CT175 t175 0 0.1f
M523 t175 na7 vdd vdd pch w=2u l=180n
M524 t175 nb5 vdd vdd pch w=2u l=180n
CT176 t176 0 0.1f
M525 t175 na7 t176 0 nch w=1u l=180n
M526 t176 nb5 0 0 nch w=1u l=180n
M527 nw88 t175 vdd vdd pch w=2u l=180n
M528 nw88 t175 0 0 nch w=1u l=180n
Cnw88 nw88 0 2f
CT177 t177 0 0.1f
M529 t177 na8 vdd vdd pch w=2u l=180n
M530 t177 nb5 vdd vdd pch w=2u l=180n
CT178 t178 0 0.1f
M531 t177 na8 t178 0 nch w=1u l=180n
M532 t178 nb5 0 0 nch w=1u l=180n
M533 nw89 t177 vdd vdd pch w=2u l=180n
M534 nw89 t177 0 0 nch w=1u l=180n
Cnw89 nw89 0 2f
CT179 t179 0 0.1f
M535 t179 na9 vdd vdd pch w=2u l=180n
M536 t179 nb5 vdd vdd pch w=2u l=180n
CT180 t180 0 0.1f
M537 t179 na9 t180 0 nch w=1u l=180n
M538 t180 nb5 0 0 nch w=1u l=180n
M539 nw90 t179 vdd vdd pch w=2u l=180n
M540 nw90 t179 0 0 nch w=1u l=180n
Cnw90 nw90 0 2f
CT181 t181 0 0.1f
M541 t181 na10 vdd vdd pch w=2u l=180n
M542 t181 nb5 vdd vdd pch w=2u l=180n
CT182 t182 0 0.1f
M543 t181 na10 t182 0 nch w=1u l=180n
M544 t182 nb5 0 0 nch w=1u l=180n
M545 nw91 t181 vdd vdd pch w=2u l=180n
M546 nw91 t181 0 0 nch w=1u l=180n
Cnw91 nw91 0 2f
CT183 t183 0 0.1f
M547 t183 na11 vdd vdd pch w=2u l=180n
M548 t183 nb5 vdd vdd pch w=2u l=180n
CT184 t184 0 0.1f
M549 t183 na11 t184 0 nch w=1u l=180n
M550 t184 nb5 0 0 nch w=1u l=180n
M551 nw92 t183 vdd vdd pch w=2u l=180n
M552 nw92 t183 0 0 nch w=1u l=180n
Cnw92 nw92 0 2f
CT185 t185 0 0.1f
M553 t185 na12 vdd vdd pch w=2u l=180n
M554 t185 nb5 vdd vdd pch w=2u l=180n
CT186 t186 0 0.1f
M555 t185 na12 t186 0 nch w=1u l=180n
M556 t186 nb5 0 0 nch w=1u l=180n
M557 nw93 t185 vdd vdd pch w=2u l=180n
M558 nw93 t185 0 0 nch w=1u l=180n
Cnw93 nw93 0 2f
CT187 t187 0 0.1f
M559 t187 na13 vdd vdd pch w=2u l=180n
M560 t187 nb5 vdd vdd pch w=2u l=180n
CT188 t188 0 0.1f
M561 t187 na13 t188 0 nch w=1u l=180n
M562 t188 nb5 0 0 nch w=1u l=180n
M563 nw94 t187 vdd vdd pch w=2u l=180n
M564 nw94 t187 0 0 nch w=1u l=180n
Cnw94 nw94 0 2f
CT189 t189 0 0.1f
M565 t189 na14 vdd vdd pch w=2u l=180n
M566 t189 nb5 vdd vdd pch w=2u l=180n
CT190 t190 0 0.1f
M567 t189 na14 t190 0 nch w=1u l=180n
M568 t190 nb5 0 0 nch w=1u l=180n
M569 nw95 t189 vdd vdd pch w=2u l=180n
M570 nw95 t189 0 0 nch w=1u l=180n
Cnw95 nw95 0 2f
CT191 t191 0 0.1f
M571 t191 na15 vdd vdd pch w=2u l=180n
M572 t191 nb5 vdd vdd pch w=2u l=180n
CT192 t192 0 0.1f
M573 t191 na15 t192 0 nch w=1u l=180n
M574 t192 nb5 0 0 nch w=1u l=180n
M575 nw96 t191 vdd vdd pch w=2u l=180n
M576 nw96 t191 0 0 nch w=1u l=180n
Cnw96 nw96 0 2f
CT193 t193 0 0.1f
M577 t193 na0 vdd vdd pch w=2u l=180n
M578 t193 nb6 vdd vdd pch w=2u l=180n
CT194 t194 0 0.1f
M579 t193 na0 t194 0 nch w=1u l=180n
M580 t194 nb6 0 0 nch w=1u l=180n
M581 nw97 t193 vdd vdd pch w=2u l=180n
M582 nw97 t193 0 0 nch w=1u l=180n
Cnw97 nw97 0 2f
CT195 t195 0 0.1f
M583 t195 na1 vdd vdd pch w=2u l=180n
M584 t195 nb6 vdd vdd pch w=2u l=180n
CT196 t196 0 0.1f
M585 t195 na1 t196 0 nch w=1u l=180n
M586 t196 nb6 0 0 nch w=1u l=180n
M587 nw98 t195 vdd vdd pch w=2u l=180n
M588 nw98 t195 0 0 nch w=1u l=180n
Cnw98 nw98 0 2f
CT197 t197 0 0.1f
M589 t197 na2 vdd vdd pch w=2u l=180n
M590 t197 nb6 vdd vdd pch w=2u l=180n
CT198 t198 0 0.1f
M591 t197 na2 t198 0 nch w=1u l=180n
M592 t198 nb6 0 0 nch w=1u l=180n
M593 nw99 t197 vdd vdd pch w=2u l=180n
M594 nw99 t197 0 0 nch w=1u l=180n
Cnw99 nw99 0 2f
CT199 t199 0 0.1f
M595 t199 na3 vdd vdd pch w=2u l=180n
M596 t199 nb6 vdd vdd pch w=2u l=180n
CT200 t200 0 0.1f
M597 t199 na3 t200 0 nch w=1u l=180n
M598 t200 nb6 0 0 nch w=1u l=180n
M599 nw100 t199 vdd vdd pch w=2u l=180n
M600 nw100 t199 0 0 nch w=1u l=180n
Cnw100 nw100 0 2f
CT201 t201 0 0.1f
M601 t201 na4 vdd vdd pch w=2u l=180n
M602 t201 nb6 vdd vdd pch w=2u l=180n
CT202 t202 0 0.1f
M603 t201 na4 t202 0 nch w=1u l=180n
M604 t202 nb6 0 0 nch w=1u l=180n
M605 nw101 t201 vdd vdd pch w=2u l=180n
M606 nw101 t201 0 0 nch w=1u l=180n
Cnw101 nw101 0 2f
CT203 t203 0 0.1f
M607 t203 na5 vdd vdd pch w=2u l=180n
M608 t203 nb6 vdd vdd pch w=2u l=180n
CT204 t204 0 0.1f
M609 t203 na5 t204 0 nch w=1u l=180n
M610 t204 nb6 0 0 nch w=1u l=180n
M611 nw102 t203 vdd vdd pch w=2u l=180n
M612 nw102 t203 0 0 nch w=1u l=180n
Cnw102 nw102 0 2f
CT205 t205 0 0.1f
M613 t205 na6 vdd vdd pch w=2u l=180n
M614 t205 nb6 vdd vdd pch w=2u l=180n
CT206 t206 0 0.1f
M615 t205 na6 t206 0 nch w=1u l=180n
M616 t206 nb6 0 0 nch w=1u l=180n
M617 nw103 t205 vdd vdd pch w=2u l=180n
M618 nw103 t205 0 0 nch w=1u l=180n
Cnw103 nw103 0 2f
CT207 t207 0 0.1f
M619 t207 na7 vdd vdd pch w=2u l=180n
M620 t207 nb6 vdd vdd pch w=2u l=180n
CT208 t208 0 0.1f
M621 t207 na7 t208 0 nch w=1u l=180n
M622 t208 nb6 0 0 nch w=1u l=180n
M623 nw104 t207 vdd vdd pch w=2u l=180n
M624 nw104 t207 0 0 nch w=1u l=180n
Cnw104 nw104 0 2f
CT209 t209 0 0.1f
M625 t209 na8 vdd vdd pch w=2u l=180n
M626 t209 nb6 vdd vdd pch w=2u l=180n
CT210 t210 0 0.1f
M627 t209 na8 t210 0 nch w=1u l=180n
M628 t210 nb6 0 0 nch w=1u l=180n
M629 nw105 t209 vdd vdd pch w=2u l=180n
M630 nw105 t209 0 0 nch w=1u l=180n
Cnw105 nw105 0 2f
CT211 t211 0 0.1f
M631 t211 na9 vdd vdd pch w=2u l=180n
M632 t211 nb6 vdd vdd pch w=2u l=180n
CT212 t212 0 0.1f
M633 t211 na9 t212 0 nch w=1u l=180n
M634 t212 nb6 0 0 nch w=1u l=180n
M635 nw106 t211 vdd vdd pch w=2u l=180n
M636 nw106 t211 0 0 nch w=1u l=180n
Cnw106 nw106 0 2f
CT213 t213 0 0.1f
M637 t213 na10 vdd vdd pch w=2u l=180n
M638 t213 nb6 vdd vdd pch w=2u l=180n
CT214 t214 0 0.1f
M639 t213 na10 t214 0 nch w=1u l=180n
M640 t214 nb6 0 0 nch w=1u l=180n
M641 nw107 t213 vdd vdd pch w=2u l=180n
M642 nw107 t213 0 0 nch w=1u l=180n
Cnw107 nw107 0 2f
CT215 t215 0 0.1f
M643 t215 na11 vdd vdd pch w=2u l=180n
M644 t215 nb6 vdd vdd pch w=2u l=180n
CT216 t216 0 0.1f
M645 t215 na11 t216 0 nch w=1u l=180n
M646 t216 nb6 0 0 nch w=1u l=180n
M647 nw108 t215 vdd vdd pch w=2u l=180n
M648 nw108 t215 0 0 nch w=1u l=180n
Cnw108 nw108 0 2f
CT217 t217 0 0.1f
M649 t217 na12 vdd vdd pch w=2u l=180n
M650 t217 nb6 vdd vdd pch w=2u l=180n
CT218 t218 0 0.1f
M651 t217 na12 t218 0 nch w=1u l=180n
M652 t218 nb6 0 0 nch w=1u l=180n
M653 nw109 t217 vdd vdd pch w=2u l=180n
M654 nw109 t217 0 0 nch w=1u l=180n
Cnw109 nw109 0 2f
CT219 t219 0 0.1f
M655 t219 na13 vdd vdd pch w=2u l=180n
M656 t219 nb6 vdd vdd pch w=2u l=180n
CT220 t220 0 0.1f
M657 t219 na13 t220 0 nch w=1u l=180n
M658 t220 nb6 0 0 nch w=1u l=180n
M659 nw110 t219 vdd vdd pch w=2u l=180n
M660 nw110 t219 0 0 nch w=1u l=180n
Cnw110 nw110 0 2f
CT221 t221 0 0.1f
M661 t221 na14 vdd vdd pch w=2u l=180n
M662 t221 nb6 vdd vdd pch w=2u l=180n
CT222 t222 0 0.1f
M663 t221 na14 t222 0 nch w=1u l=180n
M664 t222 nb6 0 0 nch w=1u l=180n
M665 nw111 t221 vdd vdd pch w=2u l=180n
M666 nw111 t221 0 0 nch w=1u l=180n
Cnw111 nw111 0 2f
CT223 t223 0 0.1f
M667 t223 na15 vdd vdd pch w=2u l=180n
M668 t223 nb6 vdd vdd pch w=2u l=180n
CT224 t224 0 0.1f
M669 t223 na15 t224 0 nch w=1u l=180n
M670 t224 nb6 0 0 nch w=1u l=180n
M671 nw112 t223 vdd vdd pch w=2u l=180n
M672 nw112 t223 0 0 nch w=1u l=180n
Cnw112 nw112 0 2f
CT225 t225 0 0.1f
M673 t225 na0 vdd vdd pch w=2u l=180n
M674 t225 nb7 vdd vdd pch w=2u l=180n
CT226 t226 0 0.1f
M675 t225 na0 t226 0 nch w=1u l=180n
M676 t226 nb7 0 0 nch w=1u l=180n
M677 nw113 t225 vdd vdd pch w=2u l=180n
M678 nw113 t225 0 0 nch w=1u l=180n
Cnw113 nw113 0 2f
CT227 t227 0 0.1f
M679 t227 na1 vdd vdd pch w=2u l=180n
M680 t227 nb7 vdd vdd pch w=2u l=180n
CT228 t228 0 0.1f
M681 t227 na1 t228 0 nch w=1u l=180n
M682 t228 nb7 0 0 nch w=1u l=180n
M683 nw114 t227 vdd vdd pch w=2u l=180n
M684 nw114 t227 0 0 nch w=1u l=180n
Cnw114 nw114 0 2f
CT229 t229 0 0.1f
M685 t229 na2 vdd vdd pch w=2u l=180n
M686 t229 nb7 vdd vdd pch w=2u l=180n
CT230 t230 0 0.1f
M687 t229 na2 t230 0 nch w=1u l=180n
M688 t230 nb7 0 0 nch w=1u l=180n
M689 nw115 t229 vdd vdd pch w=2u l=180n
M690 nw115 t229 0 0 nch w=1u l=180n
Cnw115 nw115 0 2f
CT231 t231 0 0.1f
M691 t231 na3 vdd vdd pch w=2u l=180n
M692 t231 nb7 vdd vdd pch w=2u l=180n
CT232 t232 0 0.1f
M693 t231 na3 t232 0 nch w=1u l=180n
M694 t232 nb7 0 0 nch w=1u l=180n
M695 nw116 t231 vdd vdd pch w=2u l=180n
M696 nw116 t231 0 0 nch w=1u l=180n
Cnw116 nw116 0 2f
CT233 t233 0 0.1f
M697 t233 na4 vdd vdd pch w=2u l=180n
M698 t233 nb7 vdd vdd pch w=2u l=180n
CT234 t234 0 0.1f
M699 t233 na4 t234 0 nch w=1u l=180n
M700 t234 nb7 0 0 nch w=1u l=180n
M701 nw117 t233 vdd vdd pch w=2u l=180n
M702 nw117 t233 0 0 nch w=1u l=180n
Cnw117 nw117 0 2f
CT235 t235 0 0.1f
M703 t235 na5 vdd vdd pch w=2u l=180n
M704 t235 nb7 vdd vdd pch w=2u l=180n
CT236 t236 0 0.1f
M705 t235 na5 t236 0 nch w=1u l=180n
M706 t236 nb7 0 0 nch w=1u l=180n
M707 nw118 t235 vdd vdd pch w=2u l=180n
M708 nw118 t235 0 0 nch w=1u l=180n
Cnw118 nw118 0 2f
CT237 t237 0 0.1f
M709 t237 na6 vdd vdd pch w=2u l=180n
M710 t237 nb7 vdd vdd pch w=2u l=180n
CT238 t238 0 0.1f
M711 t237 na6 t238 0 nch w=1u l=180n
M712 t238 nb7 0 0 nch w=1u l=180n
M713 nw119 t237 vdd vdd pch w=2u l=180n
M714 nw119 t237 0 0 nch w=1u l=180n
Cnw119 nw119 0 2f
CT239 t239 0 0.1f
M715 t239 na7 vdd vdd pch w=2u l=180n
M716 t239 nb7 vdd vdd pch w=2u l=180n
CT240 t240 0 0.1f
M717 t239 na7 t240 0 nch w=1u l=180n
M718 t240 nb7 0 0 nch w=1u l=180n
M719 nw120 t239 vdd vdd pch w=2u l=180n
M720 nw120 t239 0 0 nch w=1u l=180n
Cnw120 nw120 0 2f
CT241 t241 0 0.1f
M721 t241 na8 vdd vdd pch w=2u l=180n
M722 t241 nb7 vdd vdd pch w=2u l=180n
CT242 t242 0 0.1f
M723 t241 na8 t242 0 nch w=1u l=180n
M724 t242 nb7 0 0 nch w=1u l=180n
M725 nw121 t241 vdd vdd pch w=2u l=180n
M726 nw121 t241 0 0 nch w=1u l=180n
Cnw121 nw121 0 2f
CT243 t243 0 0.1f
M727 t243 na9 vdd vdd pch w=2u l=180n
M728 t243 nb7 vdd vdd pch w=2u l=180n
CT244 t244 0 0.1f
M729 t243 na9 t244 0 nch w=1u l=180n
M730 t244 nb7 0 0 nch w=1u l=180n
M731 nw122 t243 vdd vdd pch w=2u l=180n
M732 nw122 t243 0 0 nch w=1u l=180n
Cnw122 nw122 0 2f
CT245 t245 0 0.1f
M733 t245 na10 vdd vdd pch w=2u l=180n
M734 t245 nb7 vdd vdd pch w=2u l=180n
CT246 t246 0 0.1f
M735 t245 na10 t246 0 nch w=1u l=180n
M736 t246 nb7 0 0 nch w=1u l=180n
M737 nw123 t245 vdd vdd pch w=2u l=180n
M738 nw123 t245 0 0 nch w=1u l=180n
Cnw123 nw123 0 2f
CT247 t247 0 0.1f
M739 t247 na11 vdd vdd pch w=2u l=180n
M740 t247 nb7 vdd vdd pch w=2u l=180n
CT248 t248 0 0.1f
M741 t247 na11 t248 0 nch w=1u l=180n
M742 t248 nb7 0 0 nch w=1u l=180n
M743 nw124 t247 vdd vdd pch w=2u l=180n
M744 nw124 t247 0 0 nch w=1u l=180n
Cnw124 nw124 0 2f
CT249 t249 0 0.1f
M745 t249 na12 vdd vdd pch w=2u l=180n
M746 t249 nb7 vdd vdd pch w=2u l=180n
CT250 t250 0 0.1f
M747 t249 na12 t250 0 nch w=1u l=180n
M748 t250 nb7 0 0 nch w=1u l=180n
M749 nw125 t249 vdd vdd pch w=2u l=180n
M750 nw125 t249 0 0 nch w=1u l=180n
Cnw125 nw125 0 2f
CT251 t251 0 0.1f
M751 t251 na13 vdd vdd pch w=2u l=180n
M752 t251 nb7 vdd vdd pch w=2u l=180n
CT252 t252 0 0.1f
M753 t251 na13 t252 0 nch w=1u l=180n
M754 t252 nb7 0 0 nch w=1u l=180n
M755 nw126 t251 vdd vdd pch w=2u l=180n
M756 nw126 t251 0 0 nch w=1u l=180n
Cnw126 nw126 0 2f
CT253 t253 0 0.1f
M757 t253 na14 vdd vdd pch w=2u l=180n
M758 t253 nb7 vdd vdd pch w=2u l=180n
CT254 t254 0 0.1f
M759 t253 na14 t254 0 nch w=1u l=180n
M760 t254 nb7 0 0 nch w=1u l=180n
M761 nw127 t253 vdd vdd pch w=2u l=180n
M762 nw127 t253 0 0 nch w=1u l=180n
Cnw127 nw127 0 2f
CT255 t255 0 0.1f
M763 t255 na15 vdd vdd pch w=2u l=180n
M764 t255 nb7 vdd vdd pch w=2u l=180n
CT256 t256 0 0.1f
M765 t255 na15 t256 0 nch w=1u l=180n
M766 t256 nb7 0 0 nch w=1u l=180n
M767 nw128 t255 vdd vdd pch w=2u l=180n
M768 nw128 t255 0 0 nch w=1u l=180n
Cnw128 nw128 0 2f
CT257 t257 0 0.1f
M769 t257 na0 vdd vdd pch w=2u l=180n
M770 t257 nb8 vdd vdd pch w=2u l=180n
CT258 t258 0 0.1f
M771 t257 na0 t258 0 nch w=1u l=180n
M772 t258 nb8 0 0 nch w=1u l=180n
M773 nw129 t257 vdd vdd pch w=2u l=180n
M774 nw129 t257 0 0 nch w=1u l=180n
Cnw129 nw129 0 2f
CT259 t259 0 0.1f
M775 t259 na1 vdd vdd pch w=2u l=180n
M776 t259 nb8 vdd vdd pch w=2u l=180n
CT260 t260 0 0.1f
M777 t259 na1 t260 0 nch w=1u l=180n
M778 t260 nb8 0 0 nch w=1u l=180n
M779 nw130 t259 vdd vdd pch w=2u l=180n
M780 nw130 t259 0 0 nch w=1u l=180n
Cnw130 nw130 0 2f
CT261 t261 0 0.1f
M781 t261 na2 vdd vdd pch w=2u l=180n
M782 t261 nb8 vdd vdd pch w=2u l=180n
CT262 t262 0 0.1f
M783 t261 na2 t262 0 nch w=1u l=180n
M784 t262 nb8 0 0 nch w=1u l=180n
M785 nw131 t261 vdd vdd pch w=2u l=180n
M786 nw131 t261 0 0 nch w=1u l=180n
Cnw131 nw131 0 2f
CT263 t263 0 0.1f
M787 t263 na3 vdd vdd pch w=2u l=180n
M788 t263 nb8 vdd vdd pch w=2u l=180n
CT264 t264 0 0.1f
M789 t263 na3 t264 0 nch w=1u l=180n
M790 t264 nb8 0 0 nch w=1u l=180n
M791 nw132 t263 vdd vdd pch w=2u l=180n
M792 nw132 t263 0 0 nch w=1u l=180n
Cnw132 nw132 0 2f
CT265 t265 0 0.1f
M793 t265 na4 vdd vdd pch w=2u l=180n
M794 t265 nb8 vdd vdd pch w=2u l=180n
CT266 t266 0 0.1f
M795 t265 na4 t266 0 nch w=1u l=180n
M796 t266 nb8 0 0 nch w=1u l=180n
M797 nw133 t265 vdd vdd pch w=2u l=180n
M798 nw133 t265 0 0 nch w=1u l=180n
Cnw133 nw133 0 2f
CT267 t267 0 0.1f
M799 t267 na5 vdd vdd pch w=2u l=180n
M800 t267 nb8 vdd vdd pch w=2u l=180n
CT268 t268 0 0.1f
M801 t267 na5 t268 0 nch w=1u l=180n
M802 t268 nb8 0 0 nch w=1u l=180n
M803 nw134 t267 vdd vdd pch w=2u l=180n
M804 nw134 t267 0 0 nch w=1u l=180n
Cnw134 nw134 0 2f
CT269 t269 0 0.1f
M805 t269 na6 vdd vdd pch w=2u l=180n
M806 t269 nb8 vdd vdd pch w=2u l=180n
CT270 t270 0 0.1f
M807 t269 na6 t270 0 nch w=1u l=180n
M808 t270 nb8 0 0 nch w=1u l=180n
M809 nw135 t269 vdd vdd pch w=2u l=180n
M810 nw135 t269 0 0 nch w=1u l=180n
Cnw135 nw135 0 2f
CT271 t271 0 0.1f
M811 t271 na7 vdd vdd pch w=2u l=180n
M812 t271 nb8 vdd vdd pch w=2u l=180n
CT272 t272 0 0.1f
M813 t271 na7 t272 0 nch w=1u l=180n
M814 t272 nb8 0 0 nch w=1u l=180n
M815 nw136 t271 vdd vdd pch w=2u l=180n
M816 nw136 t271 0 0 nch w=1u l=180n
Cnw136 nw136 0 2f
CT273 t273 0 0.1f
M817 t273 na8 vdd vdd pch w=2u l=180n
M818 t273 nb8 vdd vdd pch w=2u l=180n
CT274 t274 0 0.1f
M819 t273 na8 t274 0 nch w=1u l=180n
M820 t274 nb8 0 0 nch w=1u l=180n
M821 nw137 t273 vdd vdd pch w=2u l=180n
M822 nw137 t273 0 0 nch w=1u l=180n
Cnw137 nw137 0 2f
CT275 t275 0 0.1f
M823 t275 na9 vdd vdd pch w=2u l=180n
M824 t275 nb8 vdd vdd pch w=2u l=180n
CT276 t276 0 0.1f
M825 t275 na9 t276 0 nch w=1u l=180n
M826 t276 nb8 0 0 nch w=1u l=180n
M827 nw138 t275 vdd vdd pch w=2u l=180n
M828 nw138 t275 0 0 nch w=1u l=180n
Cnw138 nw138 0 2f
CT277 t277 0 0.1f
M829 t277 na10 vdd vdd pch w=2u l=180n
M830 t277 nb8 vdd vdd pch w=2u l=180n
CT278 t278 0 0.1f
M831 t277 na10 t278 0 nch w=1u l=180n
M832 t278 nb8 0 0 nch w=1u l=180n
M833 nw139 t277 vdd vdd pch w=2u l=180n
M834 nw139 t277 0 0 nch w=1u l=180n
Cnw139 nw139 0 2f
CT279 t279 0 0.1f
M835 t279 na11 vdd vdd pch w=2u l=180n
M836 t279 nb8 vdd vdd pch w=2u l=180n
CT280 t280 0 0.1f
M837 t279 na11 t280 0 nch w=1u l=180n
M838 t280 nb8 0 0 nch w=1u l=180n
M839 nw140 t279 vdd vdd pch w=2u l=180n
M840 nw140 t279 0 0 nch w=1u l=180n
Cnw140 nw140 0 2f
CT281 t281 0 0.1f
M841 t281 na12 vdd vdd pch w=2u l=180n
M842 t281 nb8 vdd vdd pch w=2u l=180n
CT282 t282 0 0.1f
M843 t281 na12 t282 0 nch w=1u l=180n
M844 t282 nb8 0 0 nch w=1u l=180n
M845 nw141 t281 vdd vdd pch w=2u l=180n
M846 nw141 t281 0 0 nch w=1u l=180n
Cnw141 nw141 0 2f
CT283 t283 0 0.1f
M847 t283 na13 vdd vdd pch w=2u l=180n
M848 t283 nb8 vdd vdd pch w=2u l=180n
CT284 t284 0 0.1f
M849 t283 na13 t284 0 nch w=1u l=180n
M850 t284 nb8 0 0 nch w=1u l=180n
M851 nw142 t283 vdd vdd pch w=2u l=180n
M852 nw142 t283 0 0 nch w=1u l=180n
Cnw142 nw142 0 2f
CT285 t285 0 0.1f
M853 t285 na14 vdd vdd pch w=2u l=180n
M854 t285 nb8 vdd vdd pch w=2u l=180n
CT286 t286 0 0.1f
M855 t285 na14 t286 0 nch w=1u l=180n
M856 t286 nb8 0 0 nch w=1u l=180n
M857 nw143 t285 vdd vdd pch w=2u l=180n
M858 nw143 t285 0 0 nch w=1u l=180n
Cnw143 nw143 0 2f
CT287 t287 0 0.1f
M859 t287 na15 vdd vdd pch w=2u l=180n
M860 t287 nb8 vdd vdd pch w=2u l=180n
CT288 t288 0 0.1f
M861 t287 na15 t288 0 nch w=1u l=180n
M862 t288 nb8 0 0 nch w=1u l=180n
M863 nw144 t287 vdd vdd pch w=2u l=180n
M864 nw144 t287 0 0 nch w=1u l=180n
Cnw144 nw144 0 2f
CT289 t289 0 0.1f
M865 t289 na0 vdd vdd pch w=2u l=180n
M866 t289 nb9 vdd vdd pch w=2u l=180n
CT290 t290 0 0.1f
M867 t289 na0 t290 0 nch w=1u l=180n
M868 t290 nb9 0 0 nch w=1u l=180n
M869 nw145 t289 vdd vdd pch w=2u l=180n
M870 nw145 t289 0 0 nch w=1u l=180n
Cnw145 nw145 0 2f
CT291 t291 0 0.1f
M871 t291 na1 vdd vdd pch w=2u l=180n
M872 t291 nb9 vdd vdd pch w=2u l=180n
CT292 t292 0 0.1f
M873 t291 na1 t292 0 nch w=1u l=180n
M874 t292 nb9 0 0 nch w=1u l=180n
M875 nw146 t291 vdd vdd pch w=2u l=180n
M876 nw146 t291 0 0 nch w=1u l=180n
Cnw146 nw146 0 2f
CT293 t293 0 0.1f
M877 t293 na2 vdd vdd pch w=2u l=180n
M878 t293 nb9 vdd vdd pch w=2u l=180n
CT294 t294 0 0.1f
M879 t293 na2 t294 0 nch w=1u l=180n
M880 t294 nb9 0 0 nch w=1u l=180n
M881 nw147 t293 vdd vdd pch w=2u l=180n
M882 nw147 t293 0 0 nch w=1u l=180n
Cnw147 nw147 0 2f
CT295 t295 0 0.1f
M883 t295 na3 vdd vdd pch w=2u l=180n
M884 t295 nb9 vdd vdd pch w=2u l=180n
CT296 t296 0 0.1f
M885 t295 na3 t296 0 nch w=1u l=180n
M886 t296 nb9 0 0 nch w=1u l=180n
M887 nw148 t295 vdd vdd pch w=2u l=180n
M888 nw148 t295 0 0 nch w=1u l=180n
Cnw148 nw148 0 2f
CT297 t297 0 0.1f
M889 t297 na4 vdd vdd pch w=2u l=180n
M890 t297 nb9 vdd vdd pch w=2u l=180n
CT298 t298 0 0.1f
M891 t297 na4 t298 0 nch w=1u l=180n
M892 t298 nb9 0 0 nch w=1u l=180n
M893 nw149 t297 vdd vdd pch w=2u l=180n
M894 nw149 t297 0 0 nch w=1u l=180n
Cnw149 nw149 0 2f
CT299 t299 0 0.1f
M895 t299 na5 vdd vdd pch w=2u l=180n
M896 t299 nb9 vdd vdd pch w=2u l=180n
CT300 t300 0 0.1f
M897 t299 na5 t300 0 nch w=1u l=180n
M898 t300 nb9 0 0 nch w=1u l=180n
M899 nw150 t299 vdd vdd pch w=2u l=180n
M900 nw150 t299 0 0 nch w=1u l=180n
Cnw150 nw150 0 2f
CT301 t301 0 0.1f
M901 t301 na6 vdd vdd pch w=2u l=180n
M902 t301 nb9 vdd vdd pch w=2u l=180n
CT302 t302 0 0.1f
M903 t301 na6 t302 0 nch w=1u l=180n
M904 t302 nb9 0 0 nch w=1u l=180n
M905 nw151 t301 vdd vdd pch w=2u l=180n
M906 nw151 t301 0 0 nch w=1u l=180n
Cnw151 nw151 0 2f
CT303 t303 0 0.1f
M907 t303 na7 vdd vdd pch w=2u l=180n
M908 t303 nb9 vdd vdd pch w=2u l=180n
CT304 t304 0 0.1f
M909 t303 na7 t304 0 nch w=1u l=180n
M910 t304 nb9 0 0 nch w=1u l=180n
M911 nw152 t303 vdd vdd pch w=2u l=180n
M912 nw152 t303 0 0 nch w=1u l=180n
Cnw152 nw152 0 2f
CT305 t305 0 0.1f
M913 t305 na8 vdd vdd pch w=2u l=180n
M914 t305 nb9 vdd vdd pch w=2u l=180n
CT306 t306 0 0.1f
M915 t305 na8 t306 0 nch w=1u l=180n
M916 t306 nb9 0 0 nch w=1u l=180n
M917 nw153 t305 vdd vdd pch w=2u l=180n
M918 nw153 t305 0 0 nch w=1u l=180n
Cnw153 nw153 0 2f
CT307 t307 0 0.1f
M919 t307 na9 vdd vdd pch w=2u l=180n
M920 t307 nb9 vdd vdd pch w=2u l=180n
CT308 t308 0 0.1f
M921 t307 na9 t308 0 nch w=1u l=180n
M922 t308 nb9 0 0 nch w=1u l=180n
M923 nw154 t307 vdd vdd pch w=2u l=180n
M924 nw154 t307 0 0 nch w=1u l=180n
Cnw154 nw154 0 2f
CT309 t309 0 0.1f
M925 t309 na10 vdd vdd pch w=2u l=180n
M926 t309 nb9 vdd vdd pch w=2u l=180n
CT310 t310 0 0.1f
M927 t309 na10 t310 0 nch w=1u l=180n
M928 t310 nb9 0 0 nch w=1u l=180n
M929 nw155 t309 vdd vdd pch w=2u l=180n
M930 nw155 t309 0 0 nch w=1u l=180n
Cnw155 nw155 0 2f
CT311 t311 0 0.1f
M931 t311 na11 vdd vdd pch w=2u l=180n
M932 t311 nb9 vdd vdd pch w=2u l=180n
CT312 t312 0 0.1f
M933 t311 na11 t312 0 nch w=1u l=180n
M934 t312 nb9 0 0 nch w=1u l=180n
M935 nw156 t311 vdd vdd pch w=2u l=180n
M936 nw156 t311 0 0 nch w=1u l=180n
Cnw156 nw156 0 2f
CT313 t313 0 0.1f
M937 t313 na12 vdd vdd pch w=2u l=180n
M938 t313 nb9 vdd vdd pch w=2u l=180n
CT314 t314 0 0.1f
M939 t313 na12 t314 0 nch w=1u l=180n
M940 t314 nb9 0 0 nch w=1u l=180n
M941 nw157 t313 vdd vdd pch w=2u l=180n
M942 nw157 t313 0 0 nch w=1u l=180n
Cnw157 nw157 0 2f
CT315 t315 0 0.1f
M943 t315 na13 vdd vdd pch w=2u l=180n
M944 t315 nb9 vdd vdd pch w=2u l=180n
CT316 t316 0 0.1f
M945 t315 na13 t316 0 nch w=1u l=180n
M946 t316 nb9 0 0 nch w=1u l=180n
M947 nw158 t315 vdd vdd pch w=2u l=180n
M948 nw158 t315 0 0 nch w=1u l=180n
Cnw158 nw158 0 2f
CT317 t317 0 0.1f
M949 t317 na14 vdd vdd pch w=2u l=180n
M950 t317 nb9 vdd vdd pch w=2u l=180n
CT318 t318 0 0.1f
M951 t317 na14 t318 0 nch w=1u l=180n
M952 t318 nb9 0 0 nch w=1u l=180n
M953 nw159 t317 vdd vdd pch w=2u l=180n
M954 nw159 t317 0 0 nch w=1u l=180n
Cnw159 nw159 0 2f
CT319 t319 0 0.1f
M955 t319 na15 vdd vdd pch w=2u l=180n
M956 t319 nb9 vdd vdd pch w=2u l=180n
CT320 t320 0 0.1f
M957 t319 na15 t320 0 nch w=1u l=180n
M958 t320 nb9 0 0 nch w=1u l=180n
M959 nw160 t319 vdd vdd pch w=2u l=180n
M960 nw160 t319 0 0 nch w=1u l=180n
Cnw160 nw160 0 2f
CT321 t321 0 0.1f
M961 t321 na0 vdd vdd pch w=2u l=180n
M962 t321 nb10 vdd vdd pch w=2u l=180n
CT322 t322 0 0.1f
M963 t321 na0 t322 0 nch w=1u l=180n
M964 t322 nb10 0 0 nch w=1u l=180n
M965 nw161 t321 vdd vdd pch w=2u l=180n
M966 nw161 t321 0 0 nch w=1u l=180n
Cnw161 nw161 0 2f
CT323 t323 0 0.1f
M967 t323 na1 vdd vdd pch w=2u l=180n
M968 t323 nb10 vdd vdd pch w=2u l=180n
CT324 t324 0 0.1f
M969 t323 na1 t324 0 nch w=1u l=180n
M970 t324 nb10 0 0 nch w=1u l=180n
M971 nw162 t323 vdd vdd pch w=2u l=180n
M972 nw162 t323 0 0 nch w=1u l=180n
Cnw162 nw162 0 2f
CT325 t325 0 0.1f
M973 t325 na2 vdd vdd pch w=2u l=180n
M974 t325 nb10 vdd vdd pch w=2u l=180n
CT326 t326 0 0.1f
M975 t325 na2 t326 0 nch w=1u l=180n
M976 t326 nb10 0 0 nch w=1u l=180n
M977 nw163 t325 vdd vdd pch w=2u l=180n
M978 nw163 t325 0 0 nch w=1u l=180n
Cnw163 nw163 0 2f
CT327 t327 0 0.1f
M979 t327 na3 vdd vdd pch w=2u l=180n
M980 t327 nb10 vdd vdd pch w=2u l=180n
CT328 t328 0 0.1f
M981 t327 na3 t328 0 nch w=1u l=180n
M982 t328 nb10 0 0 nch w=1u l=180n
M983 nw164 t327 vdd vdd pch w=2u l=180n
M984 nw164 t327 0 0 nch w=1u l=180n
Cnw164 nw164 0 2f
CT329 t329 0 0.1f
M985 t329 na4 vdd vdd pch w=2u l=180n
M986 t329 nb10 vdd vdd pch w=2u l=180n
CT330 t330 0 0.1f
M987 t329 na4 t330 0 nch w=1u l=180n
M988 t330 nb10 0 0 nch w=1u l=180n
M989 nw165 t329 vdd vdd pch w=2u l=180n
M990 nw165 t329 0 0 nch w=1u l=180n
Cnw165 nw165 0 2f
CT331 t331 0 0.1f
M991 t331 na5 vdd vdd pch w=2u l=180n
M992 t331 nb10 vdd vdd pch w=2u l=180n
CT332 t332 0 0.1f
M993 t331 na5 t332 0 nch w=1u l=180n
M994 t332 nb10 0 0 nch w=1u l=180n
M995 nw166 t331 vdd vdd pch w=2u l=180n
M996 nw166 t331 0 0 nch w=1u l=180n
Cnw166 nw166 0 2f
CT333 t333 0 0.1f
M997 t333 na6 vdd vdd pch w=2u l=180n
M998 t333 nb10 vdd vdd pch w=2u l=180n
CT334 t334 0 0.1f
M999 t333 na6 t334 0 nch w=1u l=180n
M1000 t334 nb10 0 0 nch w=1u l=180n
M1001 nw167 t333 vdd vdd pch w=2u l=180n
M1002 nw167 t333 0 0 nch w=1u l=180n
Cnw167 nw167 0 2f
CT335 t335 0 0.1f
M1003 t335 na7 vdd vdd pch w=2u l=180n
M1004 t335 nb10 vdd vdd pch w=2u l=180n
CT336 t336 0 0.1f
M1005 t335 na7 t336 0 nch w=1u l=180n
M1006 t336 nb10 0 0 nch w=1u l=180n
M1007 nw168 t335 vdd vdd pch w=2u l=180n
M1008 nw168 t335 0 0 nch w=1u l=180n
Cnw168 nw168 0 2f
CT337 t337 0 0.1f
M1009 t337 na8 vdd vdd pch w=2u l=180n
M1010 t337 nb10 vdd vdd pch w=2u l=180n
CT338 t338 0 0.1f
M1011 t337 na8 t338 0 nch w=1u l=180n
M1012 t338 nb10 0 0 nch w=1u l=180n
M1013 nw169 t337 vdd vdd pch w=2u l=180n
M1014 nw169 t337 0 0 nch w=1u l=180n
Cnw169 nw169 0 2f
CT339 t339 0 0.1f
M1015 t339 na9 vdd vdd pch w=2u l=180n
M1016 t339 nb10 vdd vdd pch w=2u l=180n
CT340 t340 0 0.1f
M1017 t339 na9 t340 0 nch w=1u l=180n
M1018 t340 nb10 0 0 nch w=1u l=180n
M1019 nw170 t339 vdd vdd pch w=2u l=180n
M1020 nw170 t339 0 0 nch w=1u l=180n
Cnw170 nw170 0 2f
CT341 t341 0 0.1f
M1021 t341 na10 vdd vdd pch w=2u l=180n
M1022 t341 nb10 vdd vdd pch w=2u l=180n
CT342 t342 0 0.1f
M1023 t341 na10 t342 0 nch w=1u l=180n
M1024 t342 nb10 0 0 nch w=1u l=180n
M1025 nw171 t341 vdd vdd pch w=2u l=180n
M1026 nw171 t341 0 0 nch w=1u l=180n
Cnw171 nw171 0 2f
CT343 t343 0 0.1f
M1027 t343 na11 vdd vdd pch w=2u l=180n
M1028 t343 nb10 vdd vdd pch w=2u l=180n
CT344 t344 0 0.1f
M1029 t343 na11 t344 0 nch w=1u l=180n
M1030 t344 nb10 0 0 nch w=1u l=180n
M1031 nw172 t343 vdd vdd pch w=2u l=180n
M1032 nw172 t343 0 0 nch w=1u l=180n
Cnw172 nw172 0 2f
CT345 t345 0 0.1f
M1033 t345 na12 vdd vdd pch w=2u l=180n
M1034 t345 nb10 vdd vdd pch w=2u l=180n
CT346 t346 0 0.1f
M1035 t345 na12 t346 0 nch w=1u l=180n
M1036 t346 nb10 0 0 nch w=1u l=180n
M1037 nw173 t345 vdd vdd pch w=2u l=180n
M1038 nw173 t345 0 0 nch w=1u l=180n
Cnw173 nw173 0 2f
CT347 t347 0 0.1f
M1039 t347 na13 vdd vdd pch w=2u l=180n
M1040 t347 nb10 vdd vdd pch w=2u l=180n
CT348 t348 0 0.1f
M1041 t347 na13 t348 0 nch w=1u l=180n
M1042 t348 nb10 0 0 nch w=1u l=180n
M1043 nw174 t347 vdd vdd pch w=2u l=180n
M1044 nw174 t347 0 0 nch w=1u l=180n
Cnw174 nw174 0 2f
CT349 t349 0 0.1f
M1045 t349 na14 vdd vdd pch w=2u l=180n
M1046 t349 nb10 vdd vdd pch w=2u l=180n
CT350 t350 0 0.1f
M1047 t349 na14 t350 0 nch w=1u l=180n
M1048 t350 nb10 0 0 nch w=1u l=180n
M1049 nw175 t349 vdd vdd pch w=2u l=180n
M1050 nw175 t349 0 0 nch w=1u l=180n
Cnw175 nw175 0 2f
CT351 t351 0 0.1f
M1051 t351 na15 vdd vdd pch w=2u l=180n
M1052 t351 nb10 vdd vdd pch w=2u l=180n
CT352 t352 0 0.1f
M1053 t351 na15 t352 0 nch w=1u l=180n
M1054 t352 nb10 0 0 nch w=1u l=180n
M1055 nw176 t351 vdd vdd pch w=2u l=180n
M1056 nw176 t351 0 0 nch w=1u l=180n
Cnw176 nw176 0 2f
CT353 t353 0 0.1f
M1057 t353 na0 vdd vdd pch w=2u l=180n
M1058 t353 nb11 vdd vdd pch w=2u l=180n
CT354 t354 0 0.1f
M1059 t353 na0 t354 0 nch w=1u l=180n
M1060 t354 nb11 0 0 nch w=1u l=180n
M1061 nw177 t353 vdd vdd pch w=2u l=180n
M1062 nw177 t353 0 0 nch w=1u l=180n
Cnw177 nw177 0 2f
CT355 t355 0 0.1f
M1063 t355 na1 vdd vdd pch w=2u l=180n
M1064 t355 nb11 vdd vdd pch w=2u l=180n
CT356 t356 0 0.1f
M1065 t355 na1 t356 0 nch w=1u l=180n
M1066 t356 nb11 0 0 nch w=1u l=180n
M1067 nw178 t355 vdd vdd pch w=2u l=180n
M1068 nw178 t355 0 0 nch w=1u l=180n
Cnw178 nw178 0 2f
CT357 t357 0 0.1f
M1069 t357 na2 vdd vdd pch w=2u l=180n
M1070 t357 nb11 vdd vdd pch w=2u l=180n
CT358 t358 0 0.1f
M1071 t357 na2 t358 0 nch w=1u l=180n
M1072 t358 nb11 0 0 nch w=1u l=180n
M1073 nw179 t357 vdd vdd pch w=2u l=180n
M1074 nw179 t357 0 0 nch w=1u l=180n
Cnw179 nw179 0 2f
CT359 t359 0 0.1f
M1075 t359 na3 vdd vdd pch w=2u l=180n
M1076 t359 nb11 vdd vdd pch w=2u l=180n
CT360 t360 0 0.1f
M1077 t359 na3 t360 0 nch w=1u l=180n
M1078 t360 nb11 0 0 nch w=1u l=180n
M1079 nw180 t359 vdd vdd pch w=2u l=180n
M1080 nw180 t359 0 0 nch w=1u l=180n
Cnw180 nw180 0 2f
CT361 t361 0 0.1f
M1081 t361 na4 vdd vdd pch w=2u l=180n
M1082 t361 nb11 vdd vdd pch w=2u l=180n
CT362 t362 0 0.1f
M1083 t361 na4 t362 0 nch w=1u l=180n
M1084 t362 nb11 0 0 nch w=1u l=180n
M1085 nw181 t361 vdd vdd pch w=2u l=180n
M1086 nw181 t361 0 0 nch w=1u l=180n
Cnw181 nw181 0 2f
CT363 t363 0 0.1f
M1087 t363 na5 vdd vdd pch w=2u l=180n
M1088 t363 nb11 vdd vdd pch w=2u l=180n
CT364 t364 0 0.1f
M1089 t363 na5 t364 0 nch w=1u l=180n
M1090 t364 nb11 0 0 nch w=1u l=180n
M1091 nw182 t363 vdd vdd pch w=2u l=180n
M1092 nw182 t363 0 0 nch w=1u l=180n
Cnw182 nw182 0 2f
CT365 t365 0 0.1f
M1093 t365 na6 vdd vdd pch w=2u l=180n
M1094 t365 nb11 vdd vdd pch w=2u l=180n
CT366 t366 0 0.1f
M1095 t365 na6 t366 0 nch w=1u l=180n
M1096 t366 nb11 0 0 nch w=1u l=180n
M1097 nw183 t365 vdd vdd pch w=2u l=180n
M1098 nw183 t365 0 0 nch w=1u l=180n
Cnw183 nw183 0 2f
CT367 t367 0 0.1f
M1099 t367 na7 vdd vdd pch w=2u l=180n
M1100 t367 nb11 vdd vdd pch w=2u l=180n
CT368 t368 0 0.1f
M1101 t367 na7 t368 0 nch w=1u l=180n
M1102 t368 nb11 0 0 nch w=1u l=180n
M1103 nw184 t367 vdd vdd pch w=2u l=180n
M1104 nw184 t367 0 0 nch w=1u l=180n
Cnw184 nw184 0 2f
CT369 t369 0 0.1f
M1105 t369 na8 vdd vdd pch w=2u l=180n
M1106 t369 nb11 vdd vdd pch w=2u l=180n
CT370 t370 0 0.1f
M1107 t369 na8 t370 0 nch w=1u l=180n
M1108 t370 nb11 0 0 nch w=1u l=180n
M1109 nw185 t369 vdd vdd pch w=2u l=180n
M1110 nw185 t369 0 0 nch w=1u l=180n
Cnw185 nw185 0 2f
CT371 t371 0 0.1f
M1111 t371 na9 vdd vdd pch w=2u l=180n
M1112 t371 nb11 vdd vdd pch w=2u l=180n
CT372 t372 0 0.1f
M1113 t371 na9 t372 0 nch w=1u l=180n
M1114 t372 nb11 0 0 nch w=1u l=180n
M1115 nw186 t371 vdd vdd pch w=2u l=180n
M1116 nw186 t371 0 0 nch w=1u l=180n
Cnw186 nw186 0 2f
CT373 t373 0 0.1f
M1117 t373 na10 vdd vdd pch w=2u l=180n
M1118 t373 nb11 vdd vdd pch w=2u l=180n
CT374 t374 0 0.1f
M1119 t373 na10 t374 0 nch w=1u l=180n
M1120 t374 nb11 0 0 nch w=1u l=180n
M1121 nw187 t373 vdd vdd pch w=2u l=180n
M1122 nw187 t373 0 0 nch w=1u l=180n
Cnw187 nw187 0 2f
CT375 t375 0 0.1f
M1123 t375 na11 vdd vdd pch w=2u l=180n
M1124 t375 nb11 vdd vdd pch w=2u l=180n
CT376 t376 0 0.1f
M1125 t375 na11 t376 0 nch w=1u l=180n
M1126 t376 nb11 0 0 nch w=1u l=180n
M1127 nw188 t375 vdd vdd pch w=2u l=180n
M1128 nw188 t375 0 0 nch w=1u l=180n
Cnw188 nw188 0 2f
CT377 t377 0 0.1f
M1129 t377 na12 vdd vdd pch w=2u l=180n
M1130 t377 nb11 vdd vdd pch w=2u l=180n
CT378 t378 0 0.1f
M1131 t377 na12 t378 0 nch w=1u l=180n
M1132 t378 nb11 0 0 nch w=1u l=180n
M1133 nw189 t377 vdd vdd pch w=2u l=180n
M1134 nw189 t377 0 0 nch w=1u l=180n
Cnw189 nw189 0 2f
CT379 t379 0 0.1f
M1135 t379 na13 vdd vdd pch w=2u l=180n
M1136 t379 nb11 vdd vdd pch w=2u l=180n
CT380 t380 0 0.1f
M1137 t379 na13 t380 0 nch w=1u l=180n
M1138 t380 nb11 0 0 nch w=1u l=180n
M1139 nw190 t379 vdd vdd pch w=2u l=180n
M1140 nw190 t379 0 0 nch w=1u l=180n
Cnw190 nw190 0 2f
CT381 t381 0 0.1f
M1141 t381 na14 vdd vdd pch w=2u l=180n
M1142 t381 nb11 vdd vdd pch w=2u l=180n
CT382 t382 0 0.1f
M1143 t381 na14 t382 0 nch w=1u l=180n
M1144 t382 nb11 0 0 nch w=1u l=180n
M1145 nw191 t381 vdd vdd pch w=2u l=180n
M1146 nw191 t381 0 0 nch w=1u l=180n
Cnw191 nw191 0 2f
CT383 t383 0 0.1f
M1147 t383 na15 vdd vdd pch w=2u l=180n
M1148 t383 nb11 vdd vdd pch w=2u l=180n
CT384 t384 0 0.1f
M1149 t383 na15 t384 0 nch w=1u l=180n
M1150 t384 nb11 0 0 nch w=1u l=180n
M1151 nw192 t383 vdd vdd pch w=2u l=180n
M1152 nw192 t383 0 0 nch w=1u l=180n
Cnw192 nw192 0 2f
CT385 t385 0 0.1f
M1153 t385 na0 vdd vdd pch w=2u l=180n
M1154 t385 nb12 vdd vdd pch w=2u l=180n
CT386 t386 0 0.1f
M1155 t385 na0 t386 0 nch w=1u l=180n
M1156 t386 nb12 0 0 nch w=1u l=180n
M1157 nw193 t385 vdd vdd pch w=2u l=180n
M1158 nw193 t385 0 0 nch w=1u l=180n
Cnw193 nw193 0 2f
CT387 t387 0 0.1f
M1159 t387 na1 vdd vdd pch w=2u l=180n
M1160 t387 nb12 vdd vdd pch w=2u l=180n
CT388 t388 0 0.1f
M1161 t387 na1 t388 0 nch w=1u l=180n
M1162 t388 nb12 0 0 nch w=1u l=180n
M1163 nw194 t387 vdd vdd pch w=2u l=180n
M1164 nw194 t387 0 0 nch w=1u l=180n
Cnw194 nw194 0 2f
CT389 t389 0 0.1f
M1165 t389 na2 vdd vdd pch w=2u l=180n
M1166 t389 nb12 vdd vdd pch w=2u l=180n
CT390 t390 0 0.1f
M1167 t389 na2 t390 0 nch w=1u l=180n
M1168 t390 nb12 0 0 nch w=1u l=180n
M1169 nw195 t389 vdd vdd pch w=2u l=180n
M1170 nw195 t389 0 0 nch w=1u l=180n
Cnw195 nw195 0 2f
CT391 t391 0 0.1f
M1171 t391 na3 vdd vdd pch w=2u l=180n
M1172 t391 nb12 vdd vdd pch w=2u l=180n
CT392 t392 0 0.1f
M1173 t391 na3 t392 0 nch w=1u l=180n
M1174 t392 nb12 0 0 nch w=1u l=180n
M1175 nw196 t391 vdd vdd pch w=2u l=180n
M1176 nw196 t391 0 0 nch w=1u l=180n
Cnw196 nw196 0 2f
CT393 t393 0 0.1f
M1177 t393 na4 vdd vdd pch w=2u l=180n
M1178 t393 nb12 vdd vdd pch w=2u l=180n
CT394 t394 0 0.1f
M1179 t393 na4 t394 0 nch w=1u l=180n
M1180 t394 nb12 0 0 nch w=1u l=180n
M1181 nw197 t393 vdd vdd pch w=2u l=180n
M1182 nw197 t393 0 0 nch w=1u l=180n
Cnw197 nw197 0 2f
CT395 t395 0 0.1f
M1183 t395 na5 vdd vdd pch w=2u l=180n
M1184 t395 nb12 vdd vdd pch w=2u l=180n
CT396 t396 0 0.1f
M1185 t395 na5 t396 0 nch w=1u l=180n
M1186 t396 nb12 0 0 nch w=1u l=180n
M1187 nw198 t395 vdd vdd pch w=2u l=180n
M1188 nw198 t395 0 0 nch w=1u l=180n
Cnw198 nw198 0 2f
CT397 t397 0 0.1f
M1189 t397 na6 vdd vdd pch w=2u l=180n
M1190 t397 nb12 vdd vdd pch w=2u l=180n
CT398 t398 0 0.1f
M1191 t397 na6 t398 0 nch w=1u l=180n
M1192 t398 nb12 0 0 nch w=1u l=180n
M1193 nw199 t397 vdd vdd pch w=2u l=180n
M1194 nw199 t397 0 0 nch w=1u l=180n
Cnw199 nw199 0 2f
CT399 t399 0 0.1f
M1195 t399 na7 vdd vdd pch w=2u l=180n
M1196 t399 nb12 vdd vdd pch w=2u l=180n
CT400 t400 0 0.1f
M1197 t399 na7 t400 0 nch w=1u l=180n
M1198 t400 nb12 0 0 nch w=1u l=180n
M1199 nw200 t399 vdd vdd pch w=2u l=180n
M1200 nw200 t399 0 0 nch w=1u l=180n
Cnw200 nw200 0 2f
CT401 t401 0 0.1f
M1201 t401 na8 vdd vdd pch w=2u l=180n
M1202 t401 nb12 vdd vdd pch w=2u l=180n
CT402 t402 0 0.1f
M1203 t401 na8 t402 0 nch w=1u l=180n
M1204 t402 nb12 0 0 nch w=1u l=180n
M1205 nw201 t401 vdd vdd pch w=2u l=180n
M1206 nw201 t401 0 0 nch w=1u l=180n
Cnw201 nw201 0 2f
CT403 t403 0 0.1f
M1207 t403 na9 vdd vdd pch w=2u l=180n
M1208 t403 nb12 vdd vdd pch w=2u l=180n
CT404 t404 0 0.1f
M1209 t403 na9 t404 0 nch w=1u l=180n
M1210 t404 nb12 0 0 nch w=1u l=180n
M1211 nw202 t403 vdd vdd pch w=2u l=180n
M1212 nw202 t403 0 0 nch w=1u l=180n
Cnw202 nw202 0 2f
CT405 t405 0 0.1f
M1213 t405 na10 vdd vdd pch w=2u l=180n
M1214 t405 nb12 vdd vdd pch w=2u l=180n
CT406 t406 0 0.1f
M1215 t405 na10 t406 0 nch w=1u l=180n
M1216 t406 nb12 0 0 nch w=1u l=180n
M1217 nw203 t405 vdd vdd pch w=2u l=180n
M1218 nw203 t405 0 0 nch w=1u l=180n
Cnw203 nw203 0 2f
CT407 t407 0 0.1f
M1219 t407 na11 vdd vdd pch w=2u l=180n
M1220 t407 nb12 vdd vdd pch w=2u l=180n
CT408 t408 0 0.1f
M1221 t407 na11 t408 0 nch w=1u l=180n
M1222 t408 nb12 0 0 nch w=1u l=180n
M1223 nw204 t407 vdd vdd pch w=2u l=180n
M1224 nw204 t407 0 0 nch w=1u l=180n
Cnw204 nw204 0 2f
CT409 t409 0 0.1f
M1225 t409 na12 vdd vdd pch w=2u l=180n
M1226 t409 nb12 vdd vdd pch w=2u l=180n
CT410 t410 0 0.1f
M1227 t409 na12 t410 0 nch w=1u l=180n
M1228 t410 nb12 0 0 nch w=1u l=180n
M1229 nw205 t409 vdd vdd pch w=2u l=180n
M1230 nw205 t409 0 0 nch w=1u l=180n
Cnw205 nw205 0 2f
CT411 t411 0 0.1f
M1231 t411 na13 vdd vdd pch w=2u l=180n
M1232 t411 nb12 vdd vdd pch w=2u l=180n
CT412 t412 0 0.1f
M1233 t411 na13 t412 0 nch w=1u l=180n
M1234 t412 nb12 0 0 nch w=1u l=180n
M1235 nw206 t411 vdd vdd pch w=2u l=180n
M1236 nw206 t411 0 0 nch w=1u l=180n
Cnw206 nw206 0 2f
CT413 t413 0 0.1f
M1237 t413 na14 vdd vdd pch w=2u l=180n
M1238 t413 nb12 vdd vdd pch w=2u l=180n
CT414 t414 0 0.1f
M1239 t413 na14 t414 0 nch w=1u l=180n
M1240 t414 nb12 0 0 nch w=1u l=180n
M1241 nw207 t413 vdd vdd pch w=2u l=180n
M1242 nw207 t413 0 0 nch w=1u l=180n
Cnw207 nw207 0 2f
CT415 t415 0 0.1f
M1243 t415 na15 vdd vdd pch w=2u l=180n
M1244 t415 nb12 vdd vdd pch w=2u l=180n
CT416 t416 0 0.1f
M1245 t415 na15 t416 0 nch w=1u l=180n
M1246 t416 nb12 0 0 nch w=1u l=180n
M1247 nw208 t415 vdd vdd pch w=2u l=180n
M1248 nw208 t415 0 0 nch w=1u l=180n
Cnw208 nw208 0 2f
CT417 t417 0 0.1f
M1249 t417 na0 vdd vdd pch w=2u l=180n
M1250 t417 nb13 vdd vdd pch w=2u l=180n
CT418 t418 0 0.1f
M1251 t417 na0 t418 0 nch w=1u l=180n
M1252 t418 nb13 0 0 nch w=1u l=180n
M1253 nw209 t417 vdd vdd pch w=2u l=180n
M1254 nw209 t417 0 0 nch w=1u l=180n
Cnw209 nw209 0 2f
CT419 t419 0 0.1f
M1255 t419 na1 vdd vdd pch w=2u l=180n
M1256 t419 nb13 vdd vdd pch w=2u l=180n
CT420 t420 0 0.1f
M1257 t419 na1 t420 0 nch w=1u l=180n
M1258 t420 nb13 0 0 nch w=1u l=180n
M1259 nw210 t419 vdd vdd pch w=2u l=180n
M1260 nw210 t419 0 0 nch w=1u l=180n
Cnw210 nw210 0 2f
CT421 t421 0 0.1f
M1261 t421 na2 vdd vdd pch w=2u l=180n
M1262 t421 nb13 vdd vdd pch w=2u l=180n
CT422 t422 0 0.1f
M1263 t421 na2 t422 0 nch w=1u l=180n
M1264 t422 nb13 0 0 nch w=1u l=180n
M1265 nw211 t421 vdd vdd pch w=2u l=180n
M1266 nw211 t421 0 0 nch w=1u l=180n
Cnw211 nw211 0 2f
CT423 t423 0 0.1f
M1267 t423 na3 vdd vdd pch w=2u l=180n
M1268 t423 nb13 vdd vdd pch w=2u l=180n
CT424 t424 0 0.1f
M1269 t423 na3 t424 0 nch w=1u l=180n
M1270 t424 nb13 0 0 nch w=1u l=180n
M1271 nw212 t423 vdd vdd pch w=2u l=180n
M1272 nw212 t423 0 0 nch w=1u l=180n
Cnw212 nw212 0 2f
CT425 t425 0 0.1f
M1273 t425 na4 vdd vdd pch w=2u l=180n
M1274 t425 nb13 vdd vdd pch w=2u l=180n
CT426 t426 0 0.1f
M1275 t425 na4 t426 0 nch w=1u l=180n
M1276 t426 nb13 0 0 nch w=1u l=180n
M1277 nw213 t425 vdd vdd pch w=2u l=180n
M1278 nw213 t425 0 0 nch w=1u l=180n
Cnw213 nw213 0 2f
CT427 t427 0 0.1f
M1279 t427 na5 vdd vdd pch w=2u l=180n
M1280 t427 nb13 vdd vdd pch w=2u l=180n
CT428 t428 0 0.1f
M1281 t427 na5 t428 0 nch w=1u l=180n
M1282 t428 nb13 0 0 nch w=1u l=180n
M1283 nw214 t427 vdd vdd pch w=2u l=180n
M1284 nw214 t427 0 0 nch w=1u l=180n
Cnw214 nw214 0 2f
CT429 t429 0 0.1f
M1285 t429 na6 vdd vdd pch w=2u l=180n
M1286 t429 nb13 vdd vdd pch w=2u l=180n
CT430 t430 0 0.1f
M1287 t429 na6 t430 0 nch w=1u l=180n
M1288 t430 nb13 0 0 nch w=1u l=180n
M1289 nw215 t429 vdd vdd pch w=2u l=180n
M1290 nw215 t429 0 0 nch w=1u l=180n
Cnw215 nw215 0 2f
CT431 t431 0 0.1f
M1291 t431 na7 vdd vdd pch w=2u l=180n
M1292 t431 nb13 vdd vdd pch w=2u l=180n
CT432 t432 0 0.1f
M1293 t431 na7 t432 0 nch w=1u l=180n
M1294 t432 nb13 0 0 nch w=1u l=180n
M1295 nw216 t431 vdd vdd pch w=2u l=180n
M1296 nw216 t431 0 0 nch w=1u l=180n
Cnw216 nw216 0 2f
CT433 t433 0 0.1f
M1297 t433 na8 vdd vdd pch w=2u l=180n
M1298 t433 nb13 vdd vdd pch w=2u l=180n
CT434 t434 0 0.1f
M1299 t433 na8 t434 0 nch w=1u l=180n
M1300 t434 nb13 0 0 nch w=1u l=180n
M1301 nw217 t433 vdd vdd pch w=2u l=180n
M1302 nw217 t433 0 0 nch w=1u l=180n
Cnw217 nw217 0 2f
CT435 t435 0 0.1f
M1303 t435 na9 vdd vdd pch w=2u l=180n
M1304 t435 nb13 vdd vdd pch w=2u l=180n
CT436 t436 0 0.1f
M1305 t435 na9 t436 0 nch w=1u l=180n
M1306 t436 nb13 0 0 nch w=1u l=180n
M1307 nw218 t435 vdd vdd pch w=2u l=180n
M1308 nw218 t435 0 0 nch w=1u l=180n
Cnw218 nw218 0 2f
CT437 t437 0 0.1f
M1309 t437 na10 vdd vdd pch w=2u l=180n
M1310 t437 nb13 vdd vdd pch w=2u l=180n
CT438 t438 0 0.1f
M1311 t437 na10 t438 0 nch w=1u l=180n
M1312 t438 nb13 0 0 nch w=1u l=180n
M1313 nw219 t437 vdd vdd pch w=2u l=180n
M1314 nw219 t437 0 0 nch w=1u l=180n
Cnw219 nw219 0 2f
CT439 t439 0 0.1f
M1315 t439 na11 vdd vdd pch w=2u l=180n
M1316 t439 nb13 vdd vdd pch w=2u l=180n
CT440 t440 0 0.1f
M1317 t439 na11 t440 0 nch w=1u l=180n
M1318 t440 nb13 0 0 nch w=1u l=180n
M1319 nw220 t439 vdd vdd pch w=2u l=180n
M1320 nw220 t439 0 0 nch w=1u l=180n
Cnw220 nw220 0 2f
CT441 t441 0 0.1f
M1321 t441 na12 vdd vdd pch w=2u l=180n
M1322 t441 nb13 vdd vdd pch w=2u l=180n
CT442 t442 0 0.1f
M1323 t441 na12 t442 0 nch w=1u l=180n
M1324 t442 nb13 0 0 nch w=1u l=180n
M1325 nw221 t441 vdd vdd pch w=2u l=180n
M1326 nw221 t441 0 0 nch w=1u l=180n
Cnw221 nw221 0 2f
CT443 t443 0 0.1f
M1327 t443 na13 vdd vdd pch w=2u l=180n
M1328 t443 nb13 vdd vdd pch w=2u l=180n
CT444 t444 0 0.1f
M1329 t443 na13 t444 0 nch w=1u l=180n
M1330 t444 nb13 0 0 nch w=1u l=180n
M1331 nw222 t443 vdd vdd pch w=2u l=180n
M1332 nw222 t443 0 0 nch w=1u l=180n
Cnw222 nw222 0 2f
CT445 t445 0 0.1f
M1333 t445 na14 vdd vdd pch w=2u l=180n
M1334 t445 nb13 vdd vdd pch w=2u l=180n
CT446 t446 0 0.1f
M1335 t445 na14 t446 0 nch w=1u l=180n
M1336 t446 nb13 0 0 nch w=1u l=180n
M1337 nw223 t445 vdd vdd pch w=2u l=180n
M1338 nw223 t445 0 0 nch w=1u l=180n
Cnw223 nw223 0 2f
CT447 t447 0 0.1f
M1339 t447 na15 vdd vdd pch w=2u l=180n
M1340 t447 nb13 vdd vdd pch w=2u l=180n
CT448 t448 0 0.1f
M1341 t447 na15 t448 0 nch w=1u l=180n
M1342 t448 nb13 0 0 nch w=1u l=180n
M1343 nw224 t447 vdd vdd pch w=2u l=180n
M1344 nw224 t447 0 0 nch w=1u l=180n
Cnw224 nw224 0 2f
CT449 t449 0 0.1f
M1345 t449 na0 vdd vdd pch w=2u l=180n
M1346 t449 nb14 vdd vdd pch w=2u l=180n
CT450 t450 0 0.1f
M1347 t449 na0 t450 0 nch w=1u l=180n
M1348 t450 nb14 0 0 nch w=1u l=180n
M1349 nw225 t449 vdd vdd pch w=2u l=180n
M1350 nw225 t449 0 0 nch w=1u l=180n
Cnw225 nw225 0 2f
CT451 t451 0 0.1f
M1351 t451 na1 vdd vdd pch w=2u l=180n
M1352 t451 nb14 vdd vdd pch w=2u l=180n
CT452 t452 0 0.1f
M1353 t451 na1 t452 0 nch w=1u l=180n
M1354 t452 nb14 0 0 nch w=1u l=180n
M1355 nw226 t451 vdd vdd pch w=2u l=180n
M1356 nw226 t451 0 0 nch w=1u l=180n
Cnw226 nw226 0 2f
CT453 t453 0 0.1f
M1357 t453 na2 vdd vdd pch w=2u l=180n
M1358 t453 nb14 vdd vdd pch w=2u l=180n
CT454 t454 0 0.1f
M1359 t453 na2 t454 0 nch w=1u l=180n
M1360 t454 nb14 0 0 nch w=1u l=180n
M1361 nw227 t453 vdd vdd pch w=2u l=180n
M1362 nw227 t453 0 0 nch w=1u l=180n
Cnw227 nw227 0 2f
CT455 t455 0 0.1f
M1363 t455 na3 vdd vdd pch w=2u l=180n
M1364 t455 nb14 vdd vdd pch w=2u l=180n
CT456 t456 0 0.1f
M1365 t455 na3 t456 0 nch w=1u l=180n
M1366 t456 nb14 0 0 nch w=1u l=180n
M1367 nw228 t455 vdd vdd pch w=2u l=180n
M1368 nw228 t455 0 0 nch w=1u l=180n
Cnw228 nw228 0 2f
CT457 t457 0 0.1f
M1369 t457 na4 vdd vdd pch w=2u l=180n
M1370 t457 nb14 vdd vdd pch w=2u l=180n
CT458 t458 0 0.1f
M1371 t457 na4 t458 0 nch w=1u l=180n
M1372 t458 nb14 0 0 nch w=1u l=180n
M1373 nw229 t457 vdd vdd pch w=2u l=180n
M1374 nw229 t457 0 0 nch w=1u l=180n
Cnw229 nw229 0 2f
CT459 t459 0 0.1f
M1375 t459 na5 vdd vdd pch w=2u l=180n
M1376 t459 nb14 vdd vdd pch w=2u l=180n
CT460 t460 0 0.1f
M1377 t459 na5 t460 0 nch w=1u l=180n
M1378 t460 nb14 0 0 nch w=1u l=180n
M1379 nw230 t459 vdd vdd pch w=2u l=180n
M1380 nw230 t459 0 0 nch w=1u l=180n
Cnw230 nw230 0 2f
CT461 t461 0 0.1f
M1381 t461 na6 vdd vdd pch w=2u l=180n
M1382 t461 nb14 vdd vdd pch w=2u l=180n
CT462 t462 0 0.1f
M1383 t461 na6 t462 0 nch w=1u l=180n
M1384 t462 nb14 0 0 nch w=1u l=180n
M1385 nw231 t461 vdd vdd pch w=2u l=180n
M1386 nw231 t461 0 0 nch w=1u l=180n
Cnw231 nw231 0 2f
CT463 t463 0 0.1f
M1387 t463 na7 vdd vdd pch w=2u l=180n
M1388 t463 nb14 vdd vdd pch w=2u l=180n
CT464 t464 0 0.1f
M1389 t463 na7 t464 0 nch w=1u l=180n
M1390 t464 nb14 0 0 nch w=1u l=180n
M1391 nw232 t463 vdd vdd pch w=2u l=180n
M1392 nw232 t463 0 0 nch w=1u l=180n
Cnw232 nw232 0 2f
CT465 t465 0 0.1f
M1393 t465 na8 vdd vdd pch w=2u l=180n
M1394 t465 nb14 vdd vdd pch w=2u l=180n
CT466 t466 0 0.1f
M1395 t465 na8 t466 0 nch w=1u l=180n
M1396 t466 nb14 0 0 nch w=1u l=180n
M1397 nw233 t465 vdd vdd pch w=2u l=180n
M1398 nw233 t465 0 0 nch w=1u l=180n
Cnw233 nw233 0 2f
CT467 t467 0 0.1f
M1399 t467 na9 vdd vdd pch w=2u l=180n
M1400 t467 nb14 vdd vdd pch w=2u l=180n
CT468 t468 0 0.1f
M1401 t467 na9 t468 0 nch w=1u l=180n
M1402 t468 nb14 0 0 nch w=1u l=180n
M1403 nw234 t467 vdd vdd pch w=2u l=180n
M1404 nw234 t467 0 0 nch w=1u l=180n
Cnw234 nw234 0 2f
CT469 t469 0 0.1f
M1405 t469 na10 vdd vdd pch w=2u l=180n
M1406 t469 nb14 vdd vdd pch w=2u l=180n
CT470 t470 0 0.1f
M1407 t469 na10 t470 0 nch w=1u l=180n
M1408 t470 nb14 0 0 nch w=1u l=180n
M1409 nw235 t469 vdd vdd pch w=2u l=180n
M1410 nw235 t469 0 0 nch w=1u l=180n
Cnw235 nw235 0 2f
CT471 t471 0 0.1f
M1411 t471 na11 vdd vdd pch w=2u l=180n
M1412 t471 nb14 vdd vdd pch w=2u l=180n
CT472 t472 0 0.1f
M1413 t471 na11 t472 0 nch w=1u l=180n
M1414 t472 nb14 0 0 nch w=1u l=180n
M1415 nw236 t471 vdd vdd pch w=2u l=180n
M1416 nw236 t471 0 0 nch w=1u l=180n
Cnw236 nw236 0 2f
CT473 t473 0 0.1f
M1417 t473 na12 vdd vdd pch w=2u l=180n
M1418 t473 nb14 vdd vdd pch w=2u l=180n
CT474 t474 0 0.1f
M1419 t473 na12 t474 0 nch w=1u l=180n
M1420 t474 nb14 0 0 nch w=1u l=180n
M1421 nw237 t473 vdd vdd pch w=2u l=180n
M1422 nw237 t473 0 0 nch w=1u l=180n
Cnw237 nw237 0 2f
CT475 t475 0 0.1f
M1423 t475 na13 vdd vdd pch w=2u l=180n
M1424 t475 nb14 vdd vdd pch w=2u l=180n
CT476 t476 0 0.1f
M1425 t475 na13 t476 0 nch w=1u l=180n
M1426 t476 nb14 0 0 nch w=1u l=180n
M1427 nw238 t475 vdd vdd pch w=2u l=180n
M1428 nw238 t475 0 0 nch w=1u l=180n
Cnw238 nw238 0 2f
CT477 t477 0 0.1f
M1429 t477 na14 vdd vdd pch w=2u l=180n
M1430 t477 nb14 vdd vdd pch w=2u l=180n
CT478 t478 0 0.1f
M1431 t477 na14 t478 0 nch w=1u l=180n
M1432 t478 nb14 0 0 nch w=1u l=180n
M1433 nw239 t477 vdd vdd pch w=2u l=180n
M1434 nw239 t477 0 0 nch w=1u l=180n
Cnw239 nw239 0 2f
CT479 t479 0 0.1f
M1435 t479 na15 vdd vdd pch w=2u l=180n
M1436 t479 nb14 vdd vdd pch w=2u l=180n
CT480 t480 0 0.1f
M1437 t479 na15 t480 0 nch w=1u l=180n
M1438 t480 nb14 0 0 nch w=1u l=180n
M1439 nw240 t479 vdd vdd pch w=2u l=180n
M1440 nw240 t479 0 0 nch w=1u l=180n
Cnw240 nw240 0 2f
CT481 t481 0 0.1f
M1441 t481 na0 vdd vdd pch w=2u l=180n
M1442 t481 nb15 vdd vdd pch w=2u l=180n
CT482 t482 0 0.1f
M1443 t481 na0 t482 0 nch w=1u l=180n
M1444 t482 nb15 0 0 nch w=1u l=180n
M1445 nw241 t481 vdd vdd pch w=2u l=180n
M1446 nw241 t481 0 0 nch w=1u l=180n
Cnw241 nw241 0 2f
CT483 t483 0 0.1f
M1447 t483 na1 vdd vdd pch w=2u l=180n
M1448 t483 nb15 vdd vdd pch w=2u l=180n
CT484 t484 0 0.1f
M1449 t483 na1 t484 0 nch w=1u l=180n
M1450 t484 nb15 0 0 nch w=1u l=180n
M1451 nw242 t483 vdd vdd pch w=2u l=180n
M1452 nw242 t483 0 0 nch w=1u l=180n
Cnw242 nw242 0 2f
CT485 t485 0 0.1f
M1453 t485 na2 vdd vdd pch w=2u l=180n
M1454 t485 nb15 vdd vdd pch w=2u l=180n
CT486 t486 0 0.1f
M1455 t485 na2 t486 0 nch w=1u l=180n
M1456 t486 nb15 0 0 nch w=1u l=180n
M1457 nw243 t485 vdd vdd pch w=2u l=180n
M1458 nw243 t485 0 0 nch w=1u l=180n
Cnw243 nw243 0 2f
CT487 t487 0 0.1f
M1459 t487 na3 vdd vdd pch w=2u l=180n
M1460 t487 nb15 vdd vdd pch w=2u l=180n
CT488 t488 0 0.1f
M1461 t487 na3 t488 0 nch w=1u l=180n
M1462 t488 nb15 0 0 nch w=1u l=180n
M1463 nw244 t487 vdd vdd pch w=2u l=180n
M1464 nw244 t487 0 0 nch w=1u l=180n
Cnw244 nw244 0 2f
CT489 t489 0 0.1f
M1465 t489 na4 vdd vdd pch w=2u l=180n
M1466 t489 nb15 vdd vdd pch w=2u l=180n
CT490 t490 0 0.1f
M1467 t489 na4 t490 0 nch w=1u l=180n
M1468 t490 nb15 0 0 nch w=1u l=180n
M1469 nw245 t489 vdd vdd pch w=2u l=180n
M1470 nw245 t489 0 0 nch w=1u l=180n
Cnw245 nw245 0 2f
CT491 t491 0 0.1f
M1471 t491 na5 vdd vdd pch w=2u l=180n
M1472 t491 nb15 vdd vdd pch w=2u l=180n
CT492 t492 0 0.1f
M1473 t491 na5 t492 0 nch w=1u l=180n
M1474 t492 nb15 0 0 nch w=1u l=180n
M1475 nw246 t491 vdd vdd pch w=2u l=180n
M1476 nw246 t491 0 0 nch w=1u l=180n
Cnw246 nw246 0 2f
CT493 t493 0 0.1f
M1477 t493 na6 vdd vdd pch w=2u l=180n
M1478 t493 nb15 vdd vdd pch w=2u l=180n
CT494 t494 0 0.1f
M1479 t493 na6 t494 0 nch w=1u l=180n
M1480 t494 nb15 0 0 nch w=1u l=180n
M1481 nw247 t493 vdd vdd pch w=2u l=180n
M1482 nw247 t493 0 0 nch w=1u l=180n
Cnw247 nw247 0 2f
CT495 t495 0 0.1f
M1483 t495 na7 vdd vdd pch w=2u l=180n
M1484 t495 nb15 vdd vdd pch w=2u l=180n
CT496 t496 0 0.1f
M1485 t495 na7 t496 0 nch w=1u l=180n
M1486 t496 nb15 0 0 nch w=1u l=180n
M1487 nw248 t495 vdd vdd pch w=2u l=180n
M1488 nw248 t495 0 0 nch w=1u l=180n
Cnw248 nw248 0 2f
CT497 t497 0 0.1f
M1489 t497 na8 vdd vdd pch w=2u l=180n
M1490 t497 nb15 vdd vdd pch w=2u l=180n
CT498 t498 0 0.1f
M1491 t497 na8 t498 0 nch w=1u l=180n
M1492 t498 nb15 0 0 nch w=1u l=180n
M1493 nw249 t497 vdd vdd pch w=2u l=180n
M1494 nw249 t497 0 0 nch w=1u l=180n
Cnw249 nw249 0 2f
CT499 t499 0 0.1f
M1495 t499 na9 vdd vdd pch w=2u l=180n
M1496 t499 nb15 vdd vdd pch w=2u l=180n
CT500 t500 0 0.1f
M1497 t499 na9 t500 0 nch w=1u l=180n
M1498 t500 nb15 0 0 nch w=1u l=180n
M1499 nw250 t499 vdd vdd pch w=2u l=180n
M1500 nw250 t499 0 0 nch w=1u l=180n
Cnw250 nw250 0 2f
CT501 t501 0 0.1f
M1501 t501 na10 vdd vdd pch w=2u l=180n
M1502 t501 nb15 vdd vdd pch w=2u l=180n
CT502 t502 0 0.1f
M1503 t501 na10 t502 0 nch w=1u l=180n
M1504 t502 nb15 0 0 nch w=1u l=180n
M1505 nw251 t501 vdd vdd pch w=2u l=180n
M1506 nw251 t501 0 0 nch w=1u l=180n
Cnw251 nw251 0 2f
CT503 t503 0 0.1f
M1507 t503 na11 vdd vdd pch w=2u l=180n
M1508 t503 nb15 vdd vdd pch w=2u l=180n
CT504 t504 0 0.1f
M1509 t503 na11 t504 0 nch w=1u l=180n
M1510 t504 nb15 0 0 nch w=1u l=180n
M1511 nw252 t503 vdd vdd pch w=2u l=180n
M1512 nw252 t503 0 0 nch w=1u l=180n
Cnw252 nw252 0 2f
CT505 t505 0 0.1f
M1513 t505 na12 vdd vdd pch w=2u l=180n
M1514 t505 nb15 vdd vdd pch w=2u l=180n
CT506 t506 0 0.1f
M1515 t505 na12 t506 0 nch w=1u l=180n
M1516 t506 nb15 0 0 nch w=1u l=180n
M1517 nw253 t505 vdd vdd pch w=2u l=180n
M1518 nw253 t505 0 0 nch w=1u l=180n
Cnw253 nw253 0 2f
CT507 t507 0 0.1f
M1519 t507 na13 vdd vdd pch w=2u l=180n
M1520 t507 nb15 vdd vdd pch w=2u l=180n
CT508 t508 0 0.1f
M1521 t507 na13 t508 0 nch w=1u l=180n
M1522 t508 nb15 0 0 nch w=1u l=180n
M1523 nw254 t507 vdd vdd pch w=2u l=180n
M1524 nw254 t507 0 0 nch w=1u l=180n
Cnw254 nw254 0 2f
CT509 t509 0 0.1f
M1525 t509 na14 vdd vdd pch w=2u l=180n
M1526 t509 nb15 vdd vdd pch w=2u l=180n
CT510 t510 0 0.1f
M1527 t509 na14 t510 0 nch w=1u l=180n
M1528 t510 nb15 0 0 nch w=1u l=180n
M1529 nw255 t509 vdd vdd pch w=2u l=180n
M1530 nw255 t509 0 0 nch w=1u l=180n
Cnw255 nw255 0 2f
CT511 t511 0 0.1f
M1531 t511 na15 vdd vdd pch w=2u l=180n
M1532 t511 nb15 vdd vdd pch w=2u l=180n
CT512 t512 0 0.1f
M1533 t511 na15 t512 0 nch w=1u l=180n
M1534 t512 nb15 0 0 nch w=1u l=180n
M1535 nw256 t511 vdd vdd pch w=2u l=180n
M1536 nw256 t511 0 0 nch w=1u l=180n
Cnw256 nw256 0 2f
CT513 t513 0 0.1f
CT514 t514 0 0.1f
CT515 t515 0 0.1f
M1537 t513 nw17 vdd vdd pch w=2u l=180n
M1538 t513 nw2 vdd vdd pch w=2u l=180n
CT516 t516 0 0.1f
M1539 t513 nw17 t516 0 nch w=1u l=180n
M1540 t516 nw2 0 0 nch w=1u l=180n
M1541 t514 nw17 vdd vdd pch w=2u l=180n
M1542 t514 t513 vdd vdd pch w=2u l=180n
CT517 t517 0 0.1f
M1543 t514 nw17 t517 0 nch w=1u l=180n
M1544 t517 t513 0 0 nch w=1u l=180n
M1545 t515 nw2 vdd vdd pch w=2u l=180n
M1546 t515 t513 vdd vdd pch w=2u l=180n
CT518 t518 0 0.1f
M1547 t515 nw2 t518 0 nch w=1u l=180n
M1548 t518 t513 0 0 nch w=1u l=180n
M1549 nw257 t514 vdd vdd pch w=2u l=180n
M1550 nw257 t515 vdd vdd pch w=2u l=180n
CT519 t519 0 0.1f
M1551 nw257 t514 t519 0 nch w=1u l=180n
M1552 t519 t515 0 0 nch w=1u l=180n
Cnw257 nw257 0 2f
CT520 t520 0 0.1f
M1553 t520 nw17 vdd vdd pch w=2u l=180n
M1554 t520 nw2 vdd vdd pch w=2u l=180n
CT521 t521 0 0.1f
M1555 t520 nw17 t521 0 nch w=1u l=180n
M1556 t521 nw2 0 0 nch w=1u l=180n
M1557 nw258 t520 vdd vdd pch w=2u l=180n
M1558 nw258 t520 0 0 nch w=1u l=180n
Cnw258 nw258 0 2f
CT522 t522 0 0.1f
CT523 t523 0 0.1f
CT524 t524 0 0.1f
M1559 t522 nw18 vdd vdd pch w=2u l=180n
M1560 t522 nw3 vdd vdd pch w=2u l=180n
CT525 t525 0 0.1f
M1561 t522 nw18 t525 0 nch w=1u l=180n
M1562 t525 nw3 0 0 nch w=1u l=180n
M1563 t523 nw18 vdd vdd pch w=2u l=180n
M1564 t523 t522 vdd vdd pch w=2u l=180n
CT526 t526 0 0.1f
M1565 t523 nw18 t526 0 nch w=1u l=180n
M1566 t526 t522 0 0 nch w=1u l=180n
M1567 t524 nw3 vdd vdd pch w=2u l=180n
M1568 t524 t522 vdd vdd pch w=2u l=180n
CT527 t527 0 0.1f
M1569 t524 nw3 t527 0 nch w=1u l=180n
M1570 t527 t522 0 0 nch w=1u l=180n
M1571 nw259 t523 vdd vdd pch w=2u l=180n
M1572 nw259 t524 vdd vdd pch w=2u l=180n
CT528 t528 0 0.1f
M1573 nw259 t523 t528 0 nch w=1u l=180n
M1574 t528 t524 0 0 nch w=1u l=180n
Cnw259 nw259 0 2f
CT529 t529 0 0.1f
CT530 t530 0 0.1f
CT531 t531 0 0.1f
M1575 t529 nw259 vdd vdd pch w=2u l=180n
M1576 t529 nw258 vdd vdd pch w=2u l=180n
CT532 t532 0 0.1f
M1577 t529 nw259 t532 0 nch w=1u l=180n
M1578 t532 nw258 0 0 nch w=1u l=180n
M1579 t530 nw259 vdd vdd pch w=2u l=180n
M1580 t530 t529 vdd vdd pch w=2u l=180n
CT533 t533 0 0.1f
M1581 t530 nw259 t533 0 nch w=1u l=180n
M1582 t533 t529 0 0 nch w=1u l=180n
M1583 t531 nw258 vdd vdd pch w=2u l=180n
M1584 t531 t529 vdd vdd pch w=2u l=180n
CT534 t534 0 0.1f
M1585 t531 nw258 t534 0 nch w=1u l=180n
M1586 t534 t529 0 0 nch w=1u l=180n
M1587 nw260 t530 vdd vdd pch w=2u l=180n
M1588 nw260 t531 vdd vdd pch w=2u l=180n
CT535 t535 0 0.1f
M1589 nw260 t530 t535 0 nch w=1u l=180n
M1590 t535 t531 0 0 nch w=1u l=180n
Cnw260 nw260 0 2f
M1591 nw261 nw18 vdd vdd pch w=2u l=180n
M1592 nw261 nw3 vdd vdd pch w=2u l=180n
CT536 t536 0 0.1f
M1593 nw261 nw18 t536 0 nch w=1u l=180n
M1594 t536 nw3 0 0 nch w=1u l=180n
Cnw261 nw261 0 2f
M1595 nw262 nw259 vdd vdd pch w=2u l=180n
M1596 nw262 nw258 vdd vdd pch w=2u l=180n
CT537 t537 0 0.1f
M1597 nw262 nw259 t537 0 nch w=1u l=180n
M1598 t537 nw258 0 0 nch w=1u l=180n
Cnw262 nw262 0 2f
M1599 nw263 nw261 vdd vdd pch w=2u l=180n
M1600 nw263 nw262 vdd vdd pch w=2u l=180n
CT538 t538 0 0.1f
M1601 nw263 nw261 t538 0 nch w=1u l=180n
M1602 t538 nw262 0 0 nch w=1u l=180n
Cnw263 nw263 0 2f
CT539 t539 0 0.1f
CT540 t540 0 0.1f
CT541 t541 0 0.1f
M1603 t539 nw19 vdd vdd pch w=2u l=180n
M1604 t539 nw4 vdd vdd pch w=2u l=180n
CT542 t542 0 0.1f
M1605 t539 nw19 t542 0 nch w=1u l=180n
M1606 t542 nw4 0 0 nch w=1u l=180n
M1607 t540 nw19 vdd vdd pch w=2u l=180n
M1608 t540 t539 vdd vdd pch w=2u l=180n
CT543 t543 0 0.1f
M1609 t540 nw19 t543 0 nch w=1u l=180n
M1610 t543 t539 0 0 nch w=1u l=180n
M1611 t541 nw4 vdd vdd pch w=2u l=180n
M1612 t541 t539 vdd vdd pch w=2u l=180n
CT544 t544 0 0.1f
M1613 t541 nw4 t544 0 nch w=1u l=180n
M1614 t544 t539 0 0 nch w=1u l=180n
M1615 nw264 t540 vdd vdd pch w=2u l=180n
M1616 nw264 t541 vdd vdd pch w=2u l=180n
CT545 t545 0 0.1f
M1617 nw264 t540 t545 0 nch w=1u l=180n
M1618 t545 t541 0 0 nch w=1u l=180n
Cnw264 nw264 0 2f
CT546 t546 0 0.1f
CT547 t547 0 0.1f
CT548 t548 0 0.1f
M1619 t546 nw264 vdd vdd pch w=2u l=180n
M1620 t546 nw263 vdd vdd pch w=2u l=180n
CT549 t549 0 0.1f
M1621 t546 nw264 t549 0 nch w=1u l=180n
M1622 t549 nw263 0 0 nch w=1u l=180n
M1623 t547 nw264 vdd vdd pch w=2u l=180n
M1624 t547 t546 vdd vdd pch w=2u l=180n
CT550 t550 0 0.1f
M1625 t547 nw264 t550 0 nch w=1u l=180n
M1626 t550 t546 0 0 nch w=1u l=180n
M1627 t548 nw263 vdd vdd pch w=2u l=180n
M1628 t548 t546 vdd vdd pch w=2u l=180n
CT551 t551 0 0.1f
M1629 t548 nw263 t551 0 nch w=1u l=180n
M1630 t551 t546 0 0 nch w=1u l=180n
M1631 nw265 t547 vdd vdd pch w=2u l=180n
M1632 nw265 t548 vdd vdd pch w=2u l=180n
CT552 t552 0 0.1f
M1633 nw265 t547 t552 0 nch w=1u l=180n
M1634 t552 t548 0 0 nch w=1u l=180n
Cnw265 nw265 0 2f
M1635 nw266 nw19 vdd vdd pch w=2u l=180n
M1636 nw266 nw4 vdd vdd pch w=2u l=180n
CT553 t553 0 0.1f
M1637 nw266 nw19 t553 0 nch w=1u l=180n
M1638 t553 nw4 0 0 nch w=1u l=180n
Cnw266 nw266 0 2f
M1639 nw267 nw264 vdd vdd pch w=2u l=180n
M1640 nw267 nw263 vdd vdd pch w=2u l=180n
CT554 t554 0 0.1f
M1641 nw267 nw264 t554 0 nch w=1u l=180n
M1642 t554 nw263 0 0 nch w=1u l=180n
Cnw267 nw267 0 2f
M1643 nw268 nw266 vdd vdd pch w=2u l=180n
M1644 nw268 nw267 vdd vdd pch w=2u l=180n
CT555 t555 0 0.1f
M1645 nw268 nw266 t555 0 nch w=1u l=180n
M1646 t555 nw267 0 0 nch w=1u l=180n
Cnw268 nw268 0 2f
CT556 t556 0 0.1f
CT557 t557 0 0.1f
CT558 t558 0 0.1f
M1647 t556 nw20 vdd vdd pch w=2u l=180n
M1648 t556 nw5 vdd vdd pch w=2u l=180n
CT559 t559 0 0.1f
M1649 t556 nw20 t559 0 nch w=1u l=180n
M1650 t559 nw5 0 0 nch w=1u l=180n
M1651 t557 nw20 vdd vdd pch w=2u l=180n
M1652 t557 t556 vdd vdd pch w=2u l=180n
CT560 t560 0 0.1f
M1653 t557 nw20 t560 0 nch w=1u l=180n
M1654 t560 t556 0 0 nch w=1u l=180n
M1655 t558 nw5 vdd vdd pch w=2u l=180n
M1656 t558 t556 vdd vdd pch w=2u l=180n
CT561 t561 0 0.1f
M1657 t558 nw5 t561 0 nch w=1u l=180n
M1658 t561 t556 0 0 nch w=1u l=180n
M1659 nw269 t557 vdd vdd pch w=2u l=180n
M1660 nw269 t558 vdd vdd pch w=2u l=180n
CT562 t562 0 0.1f
M1661 nw269 t557 t562 0 nch w=1u l=180n
M1662 t562 t558 0 0 nch w=1u l=180n
Cnw269 nw269 0 2f
CT563 t563 0 0.1f
CT564 t564 0 0.1f
CT565 t565 0 0.1f
M1663 t563 nw269 vdd vdd pch w=2u l=180n
M1664 t563 nw268 vdd vdd pch w=2u l=180n
CT566 t566 0 0.1f
M1665 t563 nw269 t566 0 nch w=1u l=180n
M1666 t566 nw268 0 0 nch w=1u l=180n
M1667 t564 nw269 vdd vdd pch w=2u l=180n
M1668 t564 t563 vdd vdd pch w=2u l=180n
CT567 t567 0 0.1f
M1669 t564 nw269 t567 0 nch w=1u l=180n
M1670 t567 t563 0 0 nch w=1u l=180n
M1671 t565 nw268 vdd vdd pch w=2u l=180n
M1672 t565 t563 vdd vdd pch w=2u l=180n
CT568 t568 0 0.1f
M1673 t565 nw268 t568 0 nch w=1u l=180n
M1674 t568 t563 0 0 nch w=1u l=180n
M1675 nw270 t564 vdd vdd pch w=2u l=180n
M1676 nw270 t565 vdd vdd pch w=2u l=180n
CT569 t569 0 0.1f
M1677 nw270 t564 t569 0 nch w=1u l=180n
M1678 t569 t565 0 0 nch w=1u l=180n
Cnw270 nw270 0 2f
M1679 nw271 nw20 vdd vdd pch w=2u l=180n
M1680 nw271 nw5 vdd vdd pch w=2u l=180n
CT570 t570 0 0.1f
M1681 nw271 nw20 t570 0 nch w=1u l=180n
M1682 t570 nw5 0 0 nch w=1u l=180n
Cnw271 nw271 0 2f
M1683 nw272 nw269 vdd vdd pch w=2u l=180n
M1684 nw272 nw268 vdd vdd pch w=2u l=180n
CT571 t571 0 0.1f
M1685 nw272 nw269 t571 0 nch w=1u l=180n
M1686 t571 nw268 0 0 nch w=1u l=180n
Cnw272 nw272 0 2f
M1687 nw273 nw271 vdd vdd pch w=2u l=180n
M1688 nw273 nw272 vdd vdd pch w=2u l=180n
CT572 t572 0 0.1f
M1689 nw273 nw271 t572 0 nch w=1u l=180n
M1690 t572 nw272 0 0 nch w=1u l=180n
Cnw273 nw273 0 2f
CT573 t573 0 0.1f
CT574 t574 0 0.1f
CT575 t575 0 0.1f
M1691 t573 nw21 vdd vdd pch w=2u l=180n
M1692 t573 nw6 vdd vdd pch w=2u l=180n
CT576 t576 0 0.1f
M1693 t573 nw21 t576 0 nch w=1u l=180n
M1694 t576 nw6 0 0 nch w=1u l=180n
M1695 t574 nw21 vdd vdd pch w=2u l=180n
M1696 t574 t573 vdd vdd pch w=2u l=180n
CT577 t577 0 0.1f
M1697 t574 nw21 t577 0 nch w=1u l=180n
M1698 t577 t573 0 0 nch w=1u l=180n
M1699 t575 nw6 vdd vdd pch w=2u l=180n
M1700 t575 t573 vdd vdd pch w=2u l=180n
CT578 t578 0 0.1f
M1701 t575 nw6 t578 0 nch w=1u l=180n
M1702 t578 t573 0 0 nch w=1u l=180n
M1703 nw274 t574 vdd vdd pch w=2u l=180n
M1704 nw274 t575 vdd vdd pch w=2u l=180n
CT579 t579 0 0.1f
M1705 nw274 t574 t579 0 nch w=1u l=180n
M1706 t579 t575 0 0 nch w=1u l=180n
Cnw274 nw274 0 2f
CT580 t580 0 0.1f
CT581 t581 0 0.1f
CT582 t582 0 0.1f
M1707 t580 nw274 vdd vdd pch w=2u l=180n
M1708 t580 nw273 vdd vdd pch w=2u l=180n
CT583 t583 0 0.1f
M1709 t580 nw274 t583 0 nch w=1u l=180n
M1710 t583 nw273 0 0 nch w=1u l=180n
M1711 t581 nw274 vdd vdd pch w=2u l=180n
M1712 t581 t580 vdd vdd pch w=2u l=180n
CT584 t584 0 0.1f
M1713 t581 nw274 t584 0 nch w=1u l=180n
M1714 t584 t580 0 0 nch w=1u l=180n
M1715 t582 nw273 vdd vdd pch w=2u l=180n
M1716 t582 t580 vdd vdd pch w=2u l=180n
CT585 t585 0 0.1f
M1717 t582 nw273 t585 0 nch w=1u l=180n
M1718 t585 t580 0 0 nch w=1u l=180n
M1719 nw275 t581 vdd vdd pch w=2u l=180n
M1720 nw275 t582 vdd vdd pch w=2u l=180n
CT586 t586 0 0.1f
M1721 nw275 t581 t586 0 nch w=1u l=180n
M1722 t586 t582 0 0 nch w=1u l=180n
Cnw275 nw275 0 2f
M1723 nw276 nw21 vdd vdd pch w=2u l=180n
M1724 nw276 nw6 vdd vdd pch w=2u l=180n
CT587 t587 0 0.1f
M1725 nw276 nw21 t587 0 nch w=1u l=180n
M1726 t587 nw6 0 0 nch w=1u l=180n
Cnw276 nw276 0 2f
M1727 nw277 nw274 vdd vdd pch w=2u l=180n
M1728 nw277 nw273 vdd vdd pch w=2u l=180n
CT588 t588 0 0.1f
M1729 nw277 nw274 t588 0 nch w=1u l=180n
M1730 t588 nw273 0 0 nch w=1u l=180n
Cnw277 nw277 0 2f
M1731 nw278 nw276 vdd vdd pch w=2u l=180n
M1732 nw278 nw277 vdd vdd pch w=2u l=180n
CT589 t589 0 0.1f
M1733 nw278 nw276 t589 0 nch w=1u l=180n
M1734 t589 nw277 0 0 nch w=1u l=180n
Cnw278 nw278 0 2f
CT590 t590 0 0.1f
CT591 t591 0 0.1f
CT592 t592 0 0.1f
M1735 t590 nw22 vdd vdd pch w=2u l=180n
M1736 t590 nw7 vdd vdd pch w=2u l=180n
CT593 t593 0 0.1f
M1737 t590 nw22 t593 0 nch w=1u l=180n
M1738 t593 nw7 0 0 nch w=1u l=180n
M1739 t591 nw22 vdd vdd pch w=2u l=180n
M1740 t591 t590 vdd vdd pch w=2u l=180n
CT594 t594 0 0.1f
M1741 t591 nw22 t594 0 nch w=1u l=180n
M1742 t594 t590 0 0 nch w=1u l=180n
M1743 t592 nw7 vdd vdd pch w=2u l=180n
M1744 t592 t590 vdd vdd pch w=2u l=180n
CT595 t595 0 0.1f
M1745 t592 nw7 t595 0 nch w=1u l=180n
M1746 t595 t590 0 0 nch w=1u l=180n
M1747 nw279 t591 vdd vdd pch w=2u l=180n
M1748 nw279 t592 vdd vdd pch w=2u l=180n
CT596 t596 0 0.1f
M1749 nw279 t591 t596 0 nch w=1u l=180n
M1750 t596 t592 0 0 nch w=1u l=180n
Cnw279 nw279 0 2f
CT597 t597 0 0.1f
CT598 t598 0 0.1f
CT599 t599 0 0.1f
M1751 t597 nw279 vdd vdd pch w=2u l=180n
M1752 t597 nw278 vdd vdd pch w=2u l=180n
CT600 t600 0 0.1f
M1753 t597 nw279 t600 0 nch w=1u l=180n
M1754 t600 nw278 0 0 nch w=1u l=180n
M1755 t598 nw279 vdd vdd pch w=2u l=180n
M1756 t598 t597 vdd vdd pch w=2u l=180n
CT601 t601 0 0.1f
M1757 t598 nw279 t601 0 nch w=1u l=180n
M1758 t601 t597 0 0 nch w=1u l=180n
M1759 t599 nw278 vdd vdd pch w=2u l=180n
M1760 t599 t597 vdd vdd pch w=2u l=180n
CT602 t602 0 0.1f
M1761 t599 nw278 t602 0 nch w=1u l=180n
M1762 t602 t597 0 0 nch w=1u l=180n
M1763 nw280 t598 vdd vdd pch w=2u l=180n
M1764 nw280 t599 vdd vdd pch w=2u l=180n
CT603 t603 0 0.1f
M1765 nw280 t598 t603 0 nch w=1u l=180n
M1766 t603 t599 0 0 nch w=1u l=180n
Cnw280 nw280 0 2f
M1767 nw281 nw22 vdd vdd pch w=2u l=180n
M1768 nw281 nw7 vdd vdd pch w=2u l=180n
CT604 t604 0 0.1f
M1769 nw281 nw22 t604 0 nch w=1u l=180n
M1770 t604 nw7 0 0 nch w=1u l=180n
Cnw281 nw281 0 2f
M1771 nw282 nw279 vdd vdd pch w=2u l=180n
M1772 nw282 nw278 vdd vdd pch w=2u l=180n
CT605 t605 0 0.1f
M1773 nw282 nw279 t605 0 nch w=1u l=180n
M1774 t605 nw278 0 0 nch w=1u l=180n
Cnw282 nw282 0 2f
M1775 nw283 nw281 vdd vdd pch w=2u l=180n
M1776 nw283 nw282 vdd vdd pch w=2u l=180n
CT606 t606 0 0.1f
M1777 nw283 nw281 t606 0 nch w=1u l=180n
M1778 t606 nw282 0 0 nch w=1u l=180n
Cnw283 nw283 0 2f
CT607 t607 0 0.1f
CT608 t608 0 0.1f
CT609 t609 0 0.1f
M1779 t607 nw23 vdd vdd pch w=2u l=180n
M1780 t607 nw8 vdd vdd pch w=2u l=180n
CT610 t610 0 0.1f
M1781 t607 nw23 t610 0 nch w=1u l=180n
M1782 t610 nw8 0 0 nch w=1u l=180n
M1783 t608 nw23 vdd vdd pch w=2u l=180n
M1784 t608 t607 vdd vdd pch w=2u l=180n
CT611 t611 0 0.1f
M1785 t608 nw23 t611 0 nch w=1u l=180n
M1786 t611 t607 0 0 nch w=1u l=180n
M1787 t609 nw8 vdd vdd pch w=2u l=180n
M1788 t609 t607 vdd vdd pch w=2u l=180n
CT612 t612 0 0.1f
M1789 t609 nw8 t612 0 nch w=1u l=180n
M1790 t612 t607 0 0 nch w=1u l=180n
M1791 nw284 t608 vdd vdd pch w=2u l=180n
M1792 nw284 t609 vdd vdd pch w=2u l=180n
CT613 t613 0 0.1f
M1793 nw284 t608 t613 0 nch w=1u l=180n
M1794 t613 t609 0 0 nch w=1u l=180n
Cnw284 nw284 0 2f
CT614 t614 0 0.1f
CT615 t615 0 0.1f
CT616 t616 0 0.1f
M1795 t614 nw284 vdd vdd pch w=2u l=180n
M1796 t614 nw283 vdd vdd pch w=2u l=180n
CT617 t617 0 0.1f
M1797 t614 nw284 t617 0 nch w=1u l=180n
M1798 t617 nw283 0 0 nch w=1u l=180n
M1799 t615 nw284 vdd vdd pch w=2u l=180n
M1800 t615 t614 vdd vdd pch w=2u l=180n
CT618 t618 0 0.1f
M1801 t615 nw284 t618 0 nch w=1u l=180n
M1802 t618 t614 0 0 nch w=1u l=180n
M1803 t616 nw283 vdd vdd pch w=2u l=180n
M1804 t616 t614 vdd vdd pch w=2u l=180n
CT619 t619 0 0.1f
M1805 t616 nw283 t619 0 nch w=1u l=180n
M1806 t619 t614 0 0 nch w=1u l=180n
M1807 nw285 t615 vdd vdd pch w=2u l=180n
M1808 nw285 t616 vdd vdd pch w=2u l=180n
CT620 t620 0 0.1f
M1809 nw285 t615 t620 0 nch w=1u l=180n
M1810 t620 t616 0 0 nch w=1u l=180n
Cnw285 nw285 0 2f
M1811 nw286 nw23 vdd vdd pch w=2u l=180n
M1812 nw286 nw8 vdd vdd pch w=2u l=180n
CT621 t621 0 0.1f
M1813 nw286 nw23 t621 0 nch w=1u l=180n
M1814 t621 nw8 0 0 nch w=1u l=180n
Cnw286 nw286 0 2f
M1815 nw287 nw284 vdd vdd pch w=2u l=180n
M1816 nw287 nw283 vdd vdd pch w=2u l=180n
CT622 t622 0 0.1f
M1817 nw287 nw284 t622 0 nch w=1u l=180n
M1818 t622 nw283 0 0 nch w=1u l=180n
Cnw287 nw287 0 2f
M1819 nw288 nw286 vdd vdd pch w=2u l=180n
M1820 nw288 nw287 vdd vdd pch w=2u l=180n
CT623 t623 0 0.1f
M1821 nw288 nw286 t623 0 nch w=1u l=180n
M1822 t623 nw287 0 0 nch w=1u l=180n
Cnw288 nw288 0 2f
CT624 t624 0 0.1f
CT625 t625 0 0.1f
CT626 t626 0 0.1f
M1823 t624 nw24 vdd vdd pch w=2u l=180n
M1824 t624 nw9 vdd vdd pch w=2u l=180n
CT627 t627 0 0.1f
M1825 t624 nw24 t627 0 nch w=1u l=180n
M1826 t627 nw9 0 0 nch w=1u l=180n
M1827 t625 nw24 vdd vdd pch w=2u l=180n
M1828 t625 t624 vdd vdd pch w=2u l=180n
CT628 t628 0 0.1f
M1829 t625 nw24 t628 0 nch w=1u l=180n
M1830 t628 t624 0 0 nch w=1u l=180n
M1831 t626 nw9 vdd vdd pch w=2u l=180n
M1832 t626 t624 vdd vdd pch w=2u l=180n
CT629 t629 0 0.1f
M1833 t626 nw9 t629 0 nch w=1u l=180n
M1834 t629 t624 0 0 nch w=1u l=180n
M1835 nw289 t625 vdd vdd pch w=2u l=180n
M1836 nw289 t626 vdd vdd pch w=2u l=180n
CT630 t630 0 0.1f
M1837 nw289 t625 t630 0 nch w=1u l=180n
M1838 t630 t626 0 0 nch w=1u l=180n
Cnw289 nw289 0 2f
CT631 t631 0 0.1f
CT632 t632 0 0.1f
CT633 t633 0 0.1f
M1839 t631 nw289 vdd vdd pch w=2u l=180n
M1840 t631 nw288 vdd vdd pch w=2u l=180n
CT634 t634 0 0.1f
M1841 t631 nw289 t634 0 nch w=1u l=180n
M1842 t634 nw288 0 0 nch w=1u l=180n
M1843 t632 nw289 vdd vdd pch w=2u l=180n
M1844 t632 t631 vdd vdd pch w=2u l=180n
CT635 t635 0 0.1f
M1845 t632 nw289 t635 0 nch w=1u l=180n
M1846 t635 t631 0 0 nch w=1u l=180n
M1847 t633 nw288 vdd vdd pch w=2u l=180n
M1848 t633 t631 vdd vdd pch w=2u l=180n
CT636 t636 0 0.1f
M1849 t633 nw288 t636 0 nch w=1u l=180n
M1850 t636 t631 0 0 nch w=1u l=180n
M1851 nw290 t632 vdd vdd pch w=2u l=180n
M1852 nw290 t633 vdd vdd pch w=2u l=180n
CT637 t637 0 0.1f
M1853 nw290 t632 t637 0 nch w=1u l=180n
M1854 t637 t633 0 0 nch w=1u l=180n
Cnw290 nw290 0 2f
M1855 nw291 nw24 vdd vdd pch w=2u l=180n
M1856 nw291 nw9 vdd vdd pch w=2u l=180n
CT638 t638 0 0.1f
M1857 nw291 nw24 t638 0 nch w=1u l=180n
M1858 t638 nw9 0 0 nch w=1u l=180n
Cnw291 nw291 0 2f
M1859 nw292 nw289 vdd vdd pch w=2u l=180n
M1860 nw292 nw288 vdd vdd pch w=2u l=180n
CT639 t639 0 0.1f
M1861 nw292 nw289 t639 0 nch w=1u l=180n
M1862 t639 nw288 0 0 nch w=1u l=180n
Cnw292 nw292 0 2f
M1863 nw293 nw291 vdd vdd pch w=2u l=180n
M1864 nw293 nw292 vdd vdd pch w=2u l=180n
CT640 t640 0 0.1f
M1865 nw293 nw291 t640 0 nch w=1u l=180n
M1866 t640 nw292 0 0 nch w=1u l=180n
Cnw293 nw293 0 2f
CT641 t641 0 0.1f
CT642 t642 0 0.1f
CT643 t643 0 0.1f
M1867 t641 nw25 vdd vdd pch w=2u l=180n
M1868 t641 nw10 vdd vdd pch w=2u l=180n
CT644 t644 0 0.1f
M1869 t641 nw25 t644 0 nch w=1u l=180n
M1870 t644 nw10 0 0 nch w=1u l=180n
M1871 t642 nw25 vdd vdd pch w=2u l=180n
M1872 t642 t641 vdd vdd pch w=2u l=180n
CT645 t645 0 0.1f
M1873 t642 nw25 t645 0 nch w=1u l=180n
M1874 t645 t641 0 0 nch w=1u l=180n
M1875 t643 nw10 vdd vdd pch w=2u l=180n
M1876 t643 t641 vdd vdd pch w=2u l=180n
CT646 t646 0 0.1f
M1877 t643 nw10 t646 0 nch w=1u l=180n
M1878 t646 t641 0 0 nch w=1u l=180n
M1879 nw294 t642 vdd vdd pch w=2u l=180n
M1880 nw294 t643 vdd vdd pch w=2u l=180n
CT647 t647 0 0.1f
M1881 nw294 t642 t647 0 nch w=1u l=180n
M1882 t647 t643 0 0 nch w=1u l=180n
Cnw294 nw294 0 2f
CT648 t648 0 0.1f
CT649 t649 0 0.1f
CT650 t650 0 0.1f
M1883 t648 nw294 vdd vdd pch w=2u l=180n
M1884 t648 nw293 vdd vdd pch w=2u l=180n
CT651 t651 0 0.1f
M1885 t648 nw294 t651 0 nch w=1u l=180n
M1886 t651 nw293 0 0 nch w=1u l=180n
M1887 t649 nw294 vdd vdd pch w=2u l=180n
M1888 t649 t648 vdd vdd pch w=2u l=180n
CT652 t652 0 0.1f
M1889 t649 nw294 t652 0 nch w=1u l=180n
M1890 t652 t648 0 0 nch w=1u l=180n
M1891 t650 nw293 vdd vdd pch w=2u l=180n
M1892 t650 t648 vdd vdd pch w=2u l=180n
CT653 t653 0 0.1f
M1893 t650 nw293 t653 0 nch w=1u l=180n
M1894 t653 t648 0 0 nch w=1u l=180n
M1895 nw295 t649 vdd vdd pch w=2u l=180n
M1896 nw295 t650 vdd vdd pch w=2u l=180n
CT654 t654 0 0.1f
M1897 nw295 t649 t654 0 nch w=1u l=180n
M1898 t654 t650 0 0 nch w=1u l=180n
Cnw295 nw295 0 2f
M1899 nw296 nw25 vdd vdd pch w=2u l=180n
M1900 nw296 nw10 vdd vdd pch w=2u l=180n
CT655 t655 0 0.1f
M1901 nw296 nw25 t655 0 nch w=1u l=180n
M1902 t655 nw10 0 0 nch w=1u l=180n
Cnw296 nw296 0 2f
M1903 nw297 nw294 vdd vdd pch w=2u l=180n
M1904 nw297 nw293 vdd vdd pch w=2u l=180n
CT656 t656 0 0.1f
M1905 nw297 nw294 t656 0 nch w=1u l=180n
M1906 t656 nw293 0 0 nch w=1u l=180n
Cnw297 nw297 0 2f
M1907 nw298 nw296 vdd vdd pch w=2u l=180n
M1908 nw298 nw297 vdd vdd pch w=2u l=180n
CT657 t657 0 0.1f
M1909 nw298 nw296 t657 0 nch w=1u l=180n
M1910 t657 nw297 0 0 nch w=1u l=180n
Cnw298 nw298 0 2f
CT658 t658 0 0.1f
CT659 t659 0 0.1f
CT660 t660 0 0.1f
M1911 t658 nw26 vdd vdd pch w=2u l=180n
M1912 t658 nw11 vdd vdd pch w=2u l=180n
CT661 t661 0 0.1f
M1913 t658 nw26 t661 0 nch w=1u l=180n
M1914 t661 nw11 0 0 nch w=1u l=180n
M1915 t659 nw26 vdd vdd pch w=2u l=180n
M1916 t659 t658 vdd vdd pch w=2u l=180n
CT662 t662 0 0.1f
M1917 t659 nw26 t662 0 nch w=1u l=180n
M1918 t662 t658 0 0 nch w=1u l=180n
M1919 t660 nw11 vdd vdd pch w=2u l=180n
M1920 t660 t658 vdd vdd pch w=2u l=180n
CT663 t663 0 0.1f
M1921 t660 nw11 t663 0 nch w=1u l=180n
M1922 t663 t658 0 0 nch w=1u l=180n
M1923 nw299 t659 vdd vdd pch w=2u l=180n
M1924 nw299 t660 vdd vdd pch w=2u l=180n
CT664 t664 0 0.1f
M1925 nw299 t659 t664 0 nch w=1u l=180n
M1926 t664 t660 0 0 nch w=1u l=180n
Cnw299 nw299 0 2f
CT665 t665 0 0.1f
CT666 t666 0 0.1f
CT667 t667 0 0.1f
M1927 t665 nw299 vdd vdd pch w=2u l=180n
M1928 t665 nw298 vdd vdd pch w=2u l=180n
CT668 t668 0 0.1f
M1929 t665 nw299 t668 0 nch w=1u l=180n
M1930 t668 nw298 0 0 nch w=1u l=180n
M1931 t666 nw299 vdd vdd pch w=2u l=180n
M1932 t666 t665 vdd vdd pch w=2u l=180n
CT669 t669 0 0.1f
M1933 t666 nw299 t669 0 nch w=1u l=180n
M1934 t669 t665 0 0 nch w=1u l=180n
M1935 t667 nw298 vdd vdd pch w=2u l=180n
M1936 t667 t665 vdd vdd pch w=2u l=180n
CT670 t670 0 0.1f
M1937 t667 nw298 t670 0 nch w=1u l=180n
M1938 t670 t665 0 0 nch w=1u l=180n
M1939 nw300 t666 vdd vdd pch w=2u l=180n
M1940 nw300 t667 vdd vdd pch w=2u l=180n
CT671 t671 0 0.1f
M1941 nw300 t666 t671 0 nch w=1u l=180n
M1942 t671 t667 0 0 nch w=1u l=180n
Cnw300 nw300 0 2f
M1943 nw301 nw26 vdd vdd pch w=2u l=180n
M1944 nw301 nw11 vdd vdd pch w=2u l=180n
CT672 t672 0 0.1f
M1945 nw301 nw26 t672 0 nch w=1u l=180n
M1946 t672 nw11 0 0 nch w=1u l=180n
Cnw301 nw301 0 2f
M1947 nw302 nw299 vdd vdd pch w=2u l=180n
M1948 nw302 nw298 vdd vdd pch w=2u l=180n
CT673 t673 0 0.1f
M1949 nw302 nw299 t673 0 nch w=1u l=180n
M1950 t673 nw298 0 0 nch w=1u l=180n
Cnw302 nw302 0 2f
M1951 nw303 nw301 vdd vdd pch w=2u l=180n
M1952 nw303 nw302 vdd vdd pch w=2u l=180n
CT674 t674 0 0.1f
M1953 nw303 nw301 t674 0 nch w=1u l=180n
M1954 t674 nw302 0 0 nch w=1u l=180n
Cnw303 nw303 0 2f
CT675 t675 0 0.1f
CT676 t676 0 0.1f
CT677 t677 0 0.1f
M1955 t675 nw27 vdd vdd pch w=2u l=180n
M1956 t675 nw12 vdd vdd pch w=2u l=180n
CT678 t678 0 0.1f
M1957 t675 nw27 t678 0 nch w=1u l=180n
M1958 t678 nw12 0 0 nch w=1u l=180n
M1959 t676 nw27 vdd vdd pch w=2u l=180n
M1960 t676 t675 vdd vdd pch w=2u l=180n
CT679 t679 0 0.1f
M1961 t676 nw27 t679 0 nch w=1u l=180n
M1962 t679 t675 0 0 nch w=1u l=180n
M1963 t677 nw12 vdd vdd pch w=2u l=180n
M1964 t677 t675 vdd vdd pch w=2u l=180n
CT680 t680 0 0.1f
M1965 t677 nw12 t680 0 nch w=1u l=180n
M1966 t680 t675 0 0 nch w=1u l=180n
M1967 nw304 t676 vdd vdd pch w=2u l=180n
M1968 nw304 t677 vdd vdd pch w=2u l=180n
CT681 t681 0 0.1f
M1969 nw304 t676 t681 0 nch w=1u l=180n
M1970 t681 t677 0 0 nch w=1u l=180n
Cnw304 nw304 0 2f
CT682 t682 0 0.1f
CT683 t683 0 0.1f
CT684 t684 0 0.1f
M1971 t682 nw304 vdd vdd pch w=2u l=180n
M1972 t682 nw303 vdd vdd pch w=2u l=180n
CT685 t685 0 0.1f
M1973 t682 nw304 t685 0 nch w=1u l=180n
M1974 t685 nw303 0 0 nch w=1u l=180n
M1975 t683 nw304 vdd vdd pch w=2u l=180n
M1976 t683 t682 vdd vdd pch w=2u l=180n
CT686 t686 0 0.1f
M1977 t683 nw304 t686 0 nch w=1u l=180n
M1978 t686 t682 0 0 nch w=1u l=180n
M1979 t684 nw303 vdd vdd pch w=2u l=180n
M1980 t684 t682 vdd vdd pch w=2u l=180n
CT687 t687 0 0.1f
M1981 t684 nw303 t687 0 nch w=1u l=180n
M1982 t687 t682 0 0 nch w=1u l=180n
M1983 nw305 t683 vdd vdd pch w=2u l=180n
M1984 nw305 t684 vdd vdd pch w=2u l=180n
CT688 t688 0 0.1f
M1985 nw305 t683 t688 0 nch w=1u l=180n
M1986 t688 t684 0 0 nch w=1u l=180n
Cnw305 nw305 0 2f
M1987 nw306 nw27 vdd vdd pch w=2u l=180n
M1988 nw306 nw12 vdd vdd pch w=2u l=180n
CT689 t689 0 0.1f
M1989 nw306 nw27 t689 0 nch w=1u l=180n
M1990 t689 nw12 0 0 nch w=1u l=180n
Cnw306 nw306 0 2f
M1991 nw307 nw304 vdd vdd pch w=2u l=180n
M1992 nw307 nw303 vdd vdd pch w=2u l=180n
CT690 t690 0 0.1f
M1993 nw307 nw304 t690 0 nch w=1u l=180n
M1994 t690 nw303 0 0 nch w=1u l=180n
Cnw307 nw307 0 2f
M1995 nw308 nw306 vdd vdd pch w=2u l=180n
M1996 nw308 nw307 vdd vdd pch w=2u l=180n
CT691 t691 0 0.1f
M1997 nw308 nw306 t691 0 nch w=1u l=180n
M1998 t691 nw307 0 0 nch w=1u l=180n
Cnw308 nw308 0 2f
CT692 t692 0 0.1f
CT693 t693 0 0.1f
CT694 t694 0 0.1f
M1999 t692 nw28 vdd vdd pch w=2u l=180n
M2000 t692 nw13 vdd vdd pch w=2u l=180n
CT695 t695 0 0.1f
M2001 t692 nw28 t695 0 nch w=1u l=180n
M2002 t695 nw13 0 0 nch w=1u l=180n
M2003 t693 nw28 vdd vdd pch w=2u l=180n
M2004 t693 t692 vdd vdd pch w=2u l=180n
CT696 t696 0 0.1f
M2005 t693 nw28 t696 0 nch w=1u l=180n
M2006 t696 t692 0 0 nch w=1u l=180n
M2007 t694 nw13 vdd vdd pch w=2u l=180n
M2008 t694 t692 vdd vdd pch w=2u l=180n
CT697 t697 0 0.1f
M2009 t694 nw13 t697 0 nch w=1u l=180n
M2010 t697 t692 0 0 nch w=1u l=180n
M2011 nw309 t693 vdd vdd pch w=2u l=180n
M2012 nw309 t694 vdd vdd pch w=2u l=180n
CT698 t698 0 0.1f
M2013 nw309 t693 t698 0 nch w=1u l=180n
M2014 t698 t694 0 0 nch w=1u l=180n
Cnw309 nw309 0 2f
CT699 t699 0 0.1f
CT700 t700 0 0.1f
CT701 t701 0 0.1f
M2015 t699 nw309 vdd vdd pch w=2u l=180n
M2016 t699 nw308 vdd vdd pch w=2u l=180n
CT702 t702 0 0.1f
M2017 t699 nw309 t702 0 nch w=1u l=180n
M2018 t702 nw308 0 0 nch w=1u l=180n
M2019 t700 nw309 vdd vdd pch w=2u l=180n
M2020 t700 t699 vdd vdd pch w=2u l=180n
CT703 t703 0 0.1f
M2021 t700 nw309 t703 0 nch w=1u l=180n
M2022 t703 t699 0 0 nch w=1u l=180n
M2023 t701 nw308 vdd vdd pch w=2u l=180n
M2024 t701 t699 vdd vdd pch w=2u l=180n
CT704 t704 0 0.1f
M2025 t701 nw308 t704 0 nch w=1u l=180n
M2026 t704 t699 0 0 nch w=1u l=180n
M2027 nw310 t700 vdd vdd pch w=2u l=180n
M2028 nw310 t701 vdd vdd pch w=2u l=180n
CT705 t705 0 0.1f
M2029 nw310 t700 t705 0 nch w=1u l=180n
M2030 t705 t701 0 0 nch w=1u l=180n
Cnw310 nw310 0 2f
M2031 nw311 nw28 vdd vdd pch w=2u l=180n
M2032 nw311 nw13 vdd vdd pch w=2u l=180n
CT706 t706 0 0.1f
M2033 nw311 nw28 t706 0 nch w=1u l=180n
M2034 t706 nw13 0 0 nch w=1u l=180n
Cnw311 nw311 0 2f
M2035 nw312 nw309 vdd vdd pch w=2u l=180n
M2036 nw312 nw308 vdd vdd pch w=2u l=180n
CT707 t707 0 0.1f
M2037 nw312 nw309 t707 0 nch w=1u l=180n
M2038 t707 nw308 0 0 nch w=1u l=180n
Cnw312 nw312 0 2f
M2039 nw313 nw311 vdd vdd pch w=2u l=180n
M2040 nw313 nw312 vdd vdd pch w=2u l=180n
CT708 t708 0 0.1f
M2041 nw313 nw311 t708 0 nch w=1u l=180n
M2042 t708 nw312 0 0 nch w=1u l=180n
Cnw313 nw313 0 2f
CT709 t709 0 0.1f
CT710 t710 0 0.1f
CT711 t711 0 0.1f
M2043 t709 nw29 vdd vdd pch w=2u l=180n
M2044 t709 nw14 vdd vdd pch w=2u l=180n
CT712 t712 0 0.1f
M2045 t709 nw29 t712 0 nch w=1u l=180n
M2046 t712 nw14 0 0 nch w=1u l=180n
M2047 t710 nw29 vdd vdd pch w=2u l=180n
M2048 t710 t709 vdd vdd pch w=2u l=180n
CT713 t713 0 0.1f
M2049 t710 nw29 t713 0 nch w=1u l=180n
M2050 t713 t709 0 0 nch w=1u l=180n
M2051 t711 nw14 vdd vdd pch w=2u l=180n
M2052 t711 t709 vdd vdd pch w=2u l=180n
CT714 t714 0 0.1f
M2053 t711 nw14 t714 0 nch w=1u l=180n
M2054 t714 t709 0 0 nch w=1u l=180n
M2055 nw314 t710 vdd vdd pch w=2u l=180n
M2056 nw314 t711 vdd vdd pch w=2u l=180n
CT715 t715 0 0.1f
M2057 nw314 t710 t715 0 nch w=1u l=180n
M2058 t715 t711 0 0 nch w=1u l=180n
Cnw314 nw314 0 2f
CT716 t716 0 0.1f
CT717 t717 0 0.1f
CT718 t718 0 0.1f
M2059 t716 nw314 vdd vdd pch w=2u l=180n
M2060 t716 nw313 vdd vdd pch w=2u l=180n
CT719 t719 0 0.1f
M2061 t716 nw314 t719 0 nch w=1u l=180n
M2062 t719 nw313 0 0 nch w=1u l=180n
M2063 t717 nw314 vdd vdd pch w=2u l=180n
M2064 t717 t716 vdd vdd pch w=2u l=180n
CT720 t720 0 0.1f
M2065 t717 nw314 t720 0 nch w=1u l=180n
M2066 t720 t716 0 0 nch w=1u l=180n
M2067 t718 nw313 vdd vdd pch w=2u l=180n
M2068 t718 t716 vdd vdd pch w=2u l=180n
CT721 t721 0 0.1f
M2069 t718 nw313 t721 0 nch w=1u l=180n
M2070 t721 t716 0 0 nch w=1u l=180n
M2071 nw315 t717 vdd vdd pch w=2u l=180n
M2072 nw315 t718 vdd vdd pch w=2u l=180n
CT722 t722 0 0.1f
M2073 nw315 t717 t722 0 nch w=1u l=180n
M2074 t722 t718 0 0 nch w=1u l=180n
Cnw315 nw315 0 2f
M2075 nw316 nw29 vdd vdd pch w=2u l=180n
M2076 nw316 nw14 vdd vdd pch w=2u l=180n
CT723 t723 0 0.1f
M2077 nw316 nw29 t723 0 nch w=1u l=180n
M2078 t723 nw14 0 0 nch w=1u l=180n
Cnw316 nw316 0 2f
M2079 nw317 nw314 vdd vdd pch w=2u l=180n
M2080 nw317 nw313 vdd vdd pch w=2u l=180n
CT724 t724 0 0.1f
M2081 nw317 nw314 t724 0 nch w=1u l=180n
M2082 t724 nw313 0 0 nch w=1u l=180n
Cnw317 nw317 0 2f
M2083 nw318 nw316 vdd vdd pch w=2u l=180n
M2084 nw318 nw317 vdd vdd pch w=2u l=180n
CT725 t725 0 0.1f
M2085 nw318 nw316 t725 0 nch w=1u l=180n
M2086 t725 nw317 0 0 nch w=1u l=180n
Cnw318 nw318 0 2f
CT726 t726 0 0.1f
CT727 t727 0 0.1f
CT728 t728 0 0.1f
M2087 t726 nw30 vdd vdd pch w=2u l=180n
M2088 t726 nw15 vdd vdd pch w=2u l=180n
CT729 t729 0 0.1f
M2089 t726 nw30 t729 0 nch w=1u l=180n
M2090 t729 nw15 0 0 nch w=1u l=180n
M2091 t727 nw30 vdd vdd pch w=2u l=180n
M2092 t727 t726 vdd vdd pch w=2u l=180n
CT730 t730 0 0.1f
M2093 t727 nw30 t730 0 nch w=1u l=180n
M2094 t730 t726 0 0 nch w=1u l=180n
M2095 t728 nw15 vdd vdd pch w=2u l=180n
M2096 t728 t726 vdd vdd pch w=2u l=180n
CT731 t731 0 0.1f
M2097 t728 nw15 t731 0 nch w=1u l=180n
M2098 t731 t726 0 0 nch w=1u l=180n
M2099 nw319 t727 vdd vdd pch w=2u l=180n
M2100 nw319 t728 vdd vdd pch w=2u l=180n
CT732 t732 0 0.1f
M2101 nw319 t727 t732 0 nch w=1u l=180n
M2102 t732 t728 0 0 nch w=1u l=180n
Cnw319 nw319 0 2f
CT733 t733 0 0.1f
CT734 t734 0 0.1f
CT735 t735 0 0.1f
M2103 t733 nw319 vdd vdd pch w=2u l=180n
M2104 t733 nw318 vdd vdd pch w=2u l=180n
CT736 t736 0 0.1f
M2105 t733 nw319 t736 0 nch w=1u l=180n
M2106 t736 nw318 0 0 nch w=1u l=180n
M2107 t734 nw319 vdd vdd pch w=2u l=180n
M2108 t734 t733 vdd vdd pch w=2u l=180n
CT737 t737 0 0.1f
M2109 t734 nw319 t737 0 nch w=1u l=180n
M2110 t737 t733 0 0 nch w=1u l=180n
M2111 t735 nw318 vdd vdd pch w=2u l=180n
M2112 t735 t733 vdd vdd pch w=2u l=180n
CT738 t738 0 0.1f
M2113 t735 nw318 t738 0 nch w=1u l=180n
M2114 t738 t733 0 0 nch w=1u l=180n
M2115 nw320 t734 vdd vdd pch w=2u l=180n
M2116 nw320 t735 vdd vdd pch w=2u l=180n
CT739 t739 0 0.1f
M2117 nw320 t734 t739 0 nch w=1u l=180n
M2118 t739 t735 0 0 nch w=1u l=180n
Cnw320 nw320 0 2f
M2119 nw321 nw30 vdd vdd pch w=2u l=180n
M2120 nw321 nw15 vdd vdd pch w=2u l=180n
CT740 t740 0 0.1f
M2121 nw321 nw30 t740 0 nch w=1u l=180n
M2122 t740 nw15 0 0 nch w=1u l=180n
Cnw321 nw321 0 2f
M2123 nw322 nw319 vdd vdd pch w=2u l=180n
M2124 nw322 nw318 vdd vdd pch w=2u l=180n
CT741 t741 0 0.1f
M2125 nw322 nw319 t741 0 nch w=1u l=180n
M2126 t741 nw318 0 0 nch w=1u l=180n
Cnw322 nw322 0 2f
M2127 nw323 nw321 vdd vdd pch w=2u l=180n
M2128 nw323 nw322 vdd vdd pch w=2u l=180n
CT742 t742 0 0.1f
M2129 nw323 nw321 t742 0 nch w=1u l=180n
M2130 t742 nw322 0 0 nch w=1u l=180n
Cnw323 nw323 0 2f
CT743 t743 0 0.1f
CT744 t744 0 0.1f
CT745 t745 0 0.1f
M2131 t743 nw31 vdd vdd pch w=2u l=180n
M2132 t743 nw16 vdd vdd pch w=2u l=180n
CT746 t746 0 0.1f
M2133 t743 nw31 t746 0 nch w=1u l=180n
M2134 t746 nw16 0 0 nch w=1u l=180n
M2135 t744 nw31 vdd vdd pch w=2u l=180n
M2136 t744 t743 vdd vdd pch w=2u l=180n
CT747 t747 0 0.1f
M2137 t744 nw31 t747 0 nch w=1u l=180n
M2138 t747 t743 0 0 nch w=1u l=180n
M2139 t745 nw16 vdd vdd pch w=2u l=180n
M2140 t745 t743 vdd vdd pch w=2u l=180n
CT748 t748 0 0.1f
M2141 t745 nw16 t748 0 nch w=1u l=180n
M2142 t748 t743 0 0 nch w=1u l=180n
M2143 nw324 t744 vdd vdd pch w=2u l=180n
M2144 nw324 t745 vdd vdd pch w=2u l=180n
CT749 t749 0 0.1f
M2145 nw324 t744 t749 0 nch w=1u l=180n
M2146 t749 t745 0 0 nch w=1u l=180n
Cnw324 nw324 0 2f
CT750 t750 0 0.1f
CT751 t751 0 0.1f
CT752 t752 0 0.1f
M2147 t750 nw324 vdd vdd pch w=2u l=180n
M2148 t750 nw323 vdd vdd pch w=2u l=180n
CT753 t753 0 0.1f
M2149 t750 nw324 t753 0 nch w=1u l=180n
M2150 t753 nw323 0 0 nch w=1u l=180n
M2151 t751 nw324 vdd vdd pch w=2u l=180n
M2152 t751 t750 vdd vdd pch w=2u l=180n
CT754 t754 0 0.1f
M2153 t751 nw324 t754 0 nch w=1u l=180n
M2154 t754 t750 0 0 nch w=1u l=180n
M2155 t752 nw323 vdd vdd pch w=2u l=180n
M2156 t752 t750 vdd vdd pch w=2u l=180n
CT755 t755 0 0.1f
M2157 t752 nw323 t755 0 nch w=1u l=180n
M2158 t755 t750 0 0 nch w=1u l=180n
M2159 nw325 t751 vdd vdd pch w=2u l=180n
M2160 nw325 t752 vdd vdd pch w=2u l=180n
CT756 t756 0 0.1f
M2161 nw325 t751 t756 0 nch w=1u l=180n
M2162 t756 t752 0 0 nch w=1u l=180n
Cnw325 nw325 0 2f
M2163 nw326 nw31 vdd vdd pch w=2u l=180n
M2164 nw326 nw16 vdd vdd pch w=2u l=180n
CT757 t757 0 0.1f
M2165 nw326 nw31 t757 0 nch w=1u l=180n
M2166 t757 nw16 0 0 nch w=1u l=180n
Cnw326 nw326 0 2f
M2167 nw327 nw324 vdd vdd pch w=2u l=180n
M2168 nw327 nw323 vdd vdd pch w=2u l=180n
CT758 t758 0 0.1f
M2169 nw327 nw324 t758 0 nch w=1u l=180n
M2170 t758 nw323 0 0 nch w=1u l=180n
Cnw327 nw327 0 2f
M2171 nw328 nw326 vdd vdd pch w=2u l=180n
M2172 nw328 nw327 vdd vdd pch w=2u l=180n
CT759 t759 0 0.1f
M2173 nw328 nw326 t759 0 nch w=1u l=180n
M2174 t759 nw327 0 0 nch w=1u l=180n
Cnw328 nw328 0 2f
CT760 t760 0 0.1f
CT761 t761 0 0.1f
CT762 t762 0 0.1f
M2175 t760 nw32 vdd vdd pch w=2u l=180n
M2176 t760 nw328 vdd vdd pch w=2u l=180n
CT763 t763 0 0.1f
M2177 t760 nw32 t763 0 nch w=1u l=180n
M2178 t763 nw328 0 0 nch w=1u l=180n
M2179 t761 nw32 vdd vdd pch w=2u l=180n
M2180 t761 t760 vdd vdd pch w=2u l=180n
CT764 t764 0 0.1f
M2181 t761 nw32 t764 0 nch w=1u l=180n
M2182 t764 t760 0 0 nch w=1u l=180n
M2183 t762 nw328 vdd vdd pch w=2u l=180n
M2184 t762 t760 vdd vdd pch w=2u l=180n
CT765 t765 0 0.1f
M2185 t762 nw328 t765 0 nch w=1u l=180n
M2186 t765 t760 0 0 nch w=1u l=180n
M2187 nw329 t761 vdd vdd pch w=2u l=180n
M2188 nw329 t762 vdd vdd pch w=2u l=180n
CT766 t766 0 0.1f
M2189 nw329 t761 t766 0 nch w=1u l=180n
M2190 t766 t762 0 0 nch w=1u l=180n
Cnw329 nw329 0 2f
CT767 t767 0 0.1f
M2191 t767 nw32 vdd vdd pch w=2u l=180n
M2192 t767 nw328 vdd vdd pch w=2u l=180n
CT768 t768 0 0.1f
M2193 t767 nw32 t768 0 nch w=1u l=180n
M2194 t768 nw328 0 0 nch w=1u l=180n
M2195 nw330 t767 vdd vdd pch w=2u l=180n
M2196 nw330 t767 0 0 nch w=1u l=180n
Cnw330 nw330 0 2f
CT769 t769 0 0.1f
CT770 t770 0 0.1f
CT771 t771 0 0.1f
M2197 t769 nw33 vdd vdd pch w=2u l=180n
M2198 t769 nw260 vdd vdd pch w=2u l=180n
CT772 t772 0 0.1f
M2199 t769 nw33 t772 0 nch w=1u l=180n
M2200 t772 nw260 0 0 nch w=1u l=180n
M2201 t770 nw33 vdd vdd pch w=2u l=180n
M2202 t770 t769 vdd vdd pch w=2u l=180n
CT773 t773 0 0.1f
M2203 t770 nw33 t773 0 nch w=1u l=180n
M2204 t773 t769 0 0 nch w=1u l=180n
M2205 t771 nw260 vdd vdd pch w=2u l=180n
M2206 t771 t769 vdd vdd pch w=2u l=180n
CT774 t774 0 0.1f
M2207 t771 nw260 t774 0 nch w=1u l=180n
M2208 t774 t769 0 0 nch w=1u l=180n
M2209 nw331 t770 vdd vdd pch w=2u l=180n
M2210 nw331 t771 vdd vdd pch w=2u l=180n
CT775 t775 0 0.1f
M2211 nw331 t770 t775 0 nch w=1u l=180n
M2212 t775 t771 0 0 nch w=1u l=180n
Cnw331 nw331 0 2f
CT776 t776 0 0.1f
M2213 t776 nw33 vdd vdd pch w=2u l=180n
M2214 t776 nw260 vdd vdd pch w=2u l=180n
CT777 t777 0 0.1f
M2215 t776 nw33 t777 0 nch w=1u l=180n
M2216 t777 nw260 0 0 nch w=1u l=180n
M2217 nw332 t776 vdd vdd pch w=2u l=180n
M2218 nw332 t776 0 0 nch w=1u l=180n
Cnw332 nw332 0 2f
CT778 t778 0 0.1f
CT779 t779 0 0.1f
CT780 t780 0 0.1f
M2219 t778 nw34 vdd vdd pch w=2u l=180n
M2220 t778 nw265 vdd vdd pch w=2u l=180n
CT781 t781 0 0.1f
M2221 t778 nw34 t781 0 nch w=1u l=180n
M2222 t781 nw265 0 0 nch w=1u l=180n
M2223 t779 nw34 vdd vdd pch w=2u l=180n
M2224 t779 t778 vdd vdd pch w=2u l=180n
CT782 t782 0 0.1f
M2225 t779 nw34 t782 0 nch w=1u l=180n
M2226 t782 t778 0 0 nch w=1u l=180n
M2227 t780 nw265 vdd vdd pch w=2u l=180n
M2228 t780 t778 vdd vdd pch w=2u l=180n
CT783 t783 0 0.1f
M2229 t780 nw265 t783 0 nch w=1u l=180n
M2230 t783 t778 0 0 nch w=1u l=180n
M2231 nw333 t779 vdd vdd pch w=2u l=180n
M2232 nw333 t780 vdd vdd pch w=2u l=180n
CT784 t784 0 0.1f
M2233 nw333 t779 t784 0 nch w=1u l=180n
M2234 t784 t780 0 0 nch w=1u l=180n
Cnw333 nw333 0 2f
CT785 t785 0 0.1f
CT786 t786 0 0.1f
CT787 t787 0 0.1f
M2235 t785 nw333 vdd vdd pch w=2u l=180n
M2236 t785 nw332 vdd vdd pch w=2u l=180n
CT788 t788 0 0.1f
M2237 t785 nw333 t788 0 nch w=1u l=180n
M2238 t788 nw332 0 0 nch w=1u l=180n
M2239 t786 nw333 vdd vdd pch w=2u l=180n
M2240 t786 t785 vdd vdd pch w=2u l=180n
CT789 t789 0 0.1f
M2241 t786 nw333 t789 0 nch w=1u l=180n
M2242 t789 t785 0 0 nch w=1u l=180n
M2243 t787 nw332 vdd vdd pch w=2u l=180n
M2244 t787 t785 vdd vdd pch w=2u l=180n
CT790 t790 0 0.1f
M2245 t787 nw332 t790 0 nch w=1u l=180n
M2246 t790 t785 0 0 nch w=1u l=180n
M2247 nw334 t786 vdd vdd pch w=2u l=180n
M2248 nw334 t787 vdd vdd pch w=2u l=180n
CT791 t791 0 0.1f
M2249 nw334 t786 t791 0 nch w=1u l=180n
M2250 t791 t787 0 0 nch w=1u l=180n
Cnw334 nw334 0 2f
M2251 nw335 nw34 vdd vdd pch w=2u l=180n
M2252 nw335 nw265 vdd vdd pch w=2u l=180n
CT792 t792 0 0.1f
M2253 nw335 nw34 t792 0 nch w=1u l=180n
M2254 t792 nw265 0 0 nch w=1u l=180n
Cnw335 nw335 0 2f
M2255 nw336 nw333 vdd vdd pch w=2u l=180n
M2256 nw336 nw332 vdd vdd pch w=2u l=180n
CT793 t793 0 0.1f
M2257 nw336 nw333 t793 0 nch w=1u l=180n
M2258 t793 nw332 0 0 nch w=1u l=180n
Cnw336 nw336 0 2f
M2259 nw337 nw335 vdd vdd pch w=2u l=180n
M2260 nw337 nw336 vdd vdd pch w=2u l=180n
CT794 t794 0 0.1f
M2261 nw337 nw335 t794 0 nch w=1u l=180n
M2262 t794 nw336 0 0 nch w=1u l=180n
Cnw337 nw337 0 2f
CT795 t795 0 0.1f
CT796 t796 0 0.1f
CT797 t797 0 0.1f
M2263 t795 nw35 vdd vdd pch w=2u l=180n
M2264 t795 nw270 vdd vdd pch w=2u l=180n
CT798 t798 0 0.1f
M2265 t795 nw35 t798 0 nch w=1u l=180n
M2266 t798 nw270 0 0 nch w=1u l=180n
M2267 t796 nw35 vdd vdd pch w=2u l=180n
M2268 t796 t795 vdd vdd pch w=2u l=180n
CT799 t799 0 0.1f
M2269 t796 nw35 t799 0 nch w=1u l=180n
M2270 t799 t795 0 0 nch w=1u l=180n
M2271 t797 nw270 vdd vdd pch w=2u l=180n
M2272 t797 t795 vdd vdd pch w=2u l=180n
CT800 t800 0 0.1f
M2273 t797 nw270 t800 0 nch w=1u l=180n
M2274 t800 t795 0 0 nch w=1u l=180n
M2275 nw338 t796 vdd vdd pch w=2u l=180n
M2276 nw338 t797 vdd vdd pch w=2u l=180n
CT801 t801 0 0.1f
M2277 nw338 t796 t801 0 nch w=1u l=180n
M2278 t801 t797 0 0 nch w=1u l=180n
Cnw338 nw338 0 2f
CT802 t802 0 0.1f
CT803 t803 0 0.1f
CT804 t804 0 0.1f
M2279 t802 nw338 vdd vdd pch w=2u l=180n
M2280 t802 nw337 vdd vdd pch w=2u l=180n
CT805 t805 0 0.1f
M2281 t802 nw338 t805 0 nch w=1u l=180n
M2282 t805 nw337 0 0 nch w=1u l=180n
M2283 t803 nw338 vdd vdd pch w=2u l=180n
M2284 t803 t802 vdd vdd pch w=2u l=180n
CT806 t806 0 0.1f
M2285 t803 nw338 t806 0 nch w=1u l=180n
M2286 t806 t802 0 0 nch w=1u l=180n
M2287 t804 nw337 vdd vdd pch w=2u l=180n
M2288 t804 t802 vdd vdd pch w=2u l=180n
CT807 t807 0 0.1f
M2289 t804 nw337 t807 0 nch w=1u l=180n
M2290 t807 t802 0 0 nch w=1u l=180n
M2291 nw339 t803 vdd vdd pch w=2u l=180n
M2292 nw339 t804 vdd vdd pch w=2u l=180n
CT808 t808 0 0.1f
M2293 nw339 t803 t808 0 nch w=1u l=180n
M2294 t808 t804 0 0 nch w=1u l=180n
Cnw339 nw339 0 2f
M2295 nw340 nw35 vdd vdd pch w=2u l=180n
M2296 nw340 nw270 vdd vdd pch w=2u l=180n
CT809 t809 0 0.1f
M2297 nw340 nw35 t809 0 nch w=1u l=180n
M2298 t809 nw270 0 0 nch w=1u l=180n
Cnw340 nw340 0 2f
M2299 nw341 nw338 vdd vdd pch w=2u l=180n
M2300 nw341 nw337 vdd vdd pch w=2u l=180n
CT810 t810 0 0.1f
M2301 nw341 nw338 t810 0 nch w=1u l=180n
M2302 t810 nw337 0 0 nch w=1u l=180n
Cnw341 nw341 0 2f
M2303 nw342 nw340 vdd vdd pch w=2u l=180n
M2304 nw342 nw341 vdd vdd pch w=2u l=180n
CT811 t811 0 0.1f
M2305 nw342 nw340 t811 0 nch w=1u l=180n
M2306 t811 nw341 0 0 nch w=1u l=180n
Cnw342 nw342 0 2f
CT812 t812 0 0.1f
CT813 t813 0 0.1f
CT814 t814 0 0.1f
M2307 t812 nw36 vdd vdd pch w=2u l=180n
M2308 t812 nw275 vdd vdd pch w=2u l=180n
CT815 t815 0 0.1f
M2309 t812 nw36 t815 0 nch w=1u l=180n
M2310 t815 nw275 0 0 nch w=1u l=180n
M2311 t813 nw36 vdd vdd pch w=2u l=180n
M2312 t813 t812 vdd vdd pch w=2u l=180n
CT816 t816 0 0.1f
M2313 t813 nw36 t816 0 nch w=1u l=180n
M2314 t816 t812 0 0 nch w=1u l=180n
M2315 t814 nw275 vdd vdd pch w=2u l=180n
M2316 t814 t812 vdd vdd pch w=2u l=180n
CT817 t817 0 0.1f
M2317 t814 nw275 t817 0 nch w=1u l=180n
M2318 t817 t812 0 0 nch w=1u l=180n
M2319 nw343 t813 vdd vdd pch w=2u l=180n
M2320 nw343 t814 vdd vdd pch w=2u l=180n
CT818 t818 0 0.1f
M2321 nw343 t813 t818 0 nch w=1u l=180n
M2322 t818 t814 0 0 nch w=1u l=180n
Cnw343 nw343 0 2f
CT819 t819 0 0.1f
CT820 t820 0 0.1f
CT821 t821 0 0.1f
M2323 t819 nw343 vdd vdd pch w=2u l=180n
M2324 t819 nw342 vdd vdd pch w=2u l=180n
CT822 t822 0 0.1f
M2325 t819 nw343 t822 0 nch w=1u l=180n
M2326 t822 nw342 0 0 nch w=1u l=180n
M2327 t820 nw343 vdd vdd pch w=2u l=180n
M2328 t820 t819 vdd vdd pch w=2u l=180n
CT823 t823 0 0.1f
M2329 t820 nw343 t823 0 nch w=1u l=180n
M2330 t823 t819 0 0 nch w=1u l=180n
M2331 t821 nw342 vdd vdd pch w=2u l=180n
M2332 t821 t819 vdd vdd pch w=2u l=180n
CT824 t824 0 0.1f
M2333 t821 nw342 t824 0 nch w=1u l=180n
M2334 t824 t819 0 0 nch w=1u l=180n
M2335 nw344 t820 vdd vdd pch w=2u l=180n
M2336 nw344 t821 vdd vdd pch w=2u l=180n
CT825 t825 0 0.1f
M2337 nw344 t820 t825 0 nch w=1u l=180n
M2338 t825 t821 0 0 nch w=1u l=180n
Cnw344 nw344 0 2f
M2339 nw345 nw36 vdd vdd pch w=2u l=180n
M2340 nw345 nw275 vdd vdd pch w=2u l=180n
CT826 t826 0 0.1f
M2341 nw345 nw36 t826 0 nch w=1u l=180n
M2342 t826 nw275 0 0 nch w=1u l=180n
Cnw345 nw345 0 2f
M2343 nw346 nw343 vdd vdd pch w=2u l=180n
M2344 nw346 nw342 vdd vdd pch w=2u l=180n
CT827 t827 0 0.1f
M2345 nw346 nw343 t827 0 nch w=1u l=180n
M2346 t827 nw342 0 0 nch w=1u l=180n
Cnw346 nw346 0 2f
M2347 nw347 nw345 vdd vdd pch w=2u l=180n
M2348 nw347 nw346 vdd vdd pch w=2u l=180n
CT828 t828 0 0.1f
M2349 nw347 nw345 t828 0 nch w=1u l=180n
M2350 t828 nw346 0 0 nch w=1u l=180n
Cnw347 nw347 0 2f
CT829 t829 0 0.1f
CT830 t830 0 0.1f
CT831 t831 0 0.1f
M2351 t829 nw37 vdd vdd pch w=2u l=180n
M2352 t829 nw280 vdd vdd pch w=2u l=180n
CT832 t832 0 0.1f
M2353 t829 nw37 t832 0 nch w=1u l=180n
M2354 t832 nw280 0 0 nch w=1u l=180n
M2355 t830 nw37 vdd vdd pch w=2u l=180n
M2356 t830 t829 vdd vdd pch w=2u l=180n
CT833 t833 0 0.1f
M2357 t830 nw37 t833 0 nch w=1u l=180n
M2358 t833 t829 0 0 nch w=1u l=180n
M2359 t831 nw280 vdd vdd pch w=2u l=180n
M2360 t831 t829 vdd vdd pch w=2u l=180n
CT834 t834 0 0.1f
M2361 t831 nw280 t834 0 nch w=1u l=180n
M2362 t834 t829 0 0 nch w=1u l=180n
M2363 nw348 t830 vdd vdd pch w=2u l=180n
M2364 nw348 t831 vdd vdd pch w=2u l=180n
CT835 t835 0 0.1f
M2365 nw348 t830 t835 0 nch w=1u l=180n
M2366 t835 t831 0 0 nch w=1u l=180n
Cnw348 nw348 0 2f
CT836 t836 0 0.1f
CT837 t837 0 0.1f
CT838 t838 0 0.1f
M2367 t836 nw348 vdd vdd pch w=2u l=180n
M2368 t836 nw347 vdd vdd pch w=2u l=180n
CT839 t839 0 0.1f
M2369 t836 nw348 t839 0 nch w=1u l=180n
M2370 t839 nw347 0 0 nch w=1u l=180n
M2371 t837 nw348 vdd vdd pch w=2u l=180n
M2372 t837 t836 vdd vdd pch w=2u l=180n
CT840 t840 0 0.1f
M2373 t837 nw348 t840 0 nch w=1u l=180n
M2374 t840 t836 0 0 nch w=1u l=180n
M2375 t838 nw347 vdd vdd pch w=2u l=180n
M2376 t838 t836 vdd vdd pch w=2u l=180n
CT841 t841 0 0.1f
M2377 t838 nw347 t841 0 nch w=1u l=180n
M2378 t841 t836 0 0 nch w=1u l=180n
M2379 nw349 t837 vdd vdd pch w=2u l=180n
M2380 nw349 t838 vdd vdd pch w=2u l=180n
CT842 t842 0 0.1f
M2381 nw349 t837 t842 0 nch w=1u l=180n
M2382 t842 t838 0 0 nch w=1u l=180n
Cnw349 nw349 0 2f
M2383 nw350 nw37 vdd vdd pch w=2u l=180n
M2384 nw350 nw280 vdd vdd pch w=2u l=180n
CT843 t843 0 0.1f
M2385 nw350 nw37 t843 0 nch w=1u l=180n
M2386 t843 nw280 0 0 nch w=1u l=180n
Cnw350 nw350 0 2f
M2387 nw351 nw348 vdd vdd pch w=2u l=180n
M2388 nw351 nw347 vdd vdd pch w=2u l=180n
CT844 t844 0 0.1f
M2389 nw351 nw348 t844 0 nch w=1u l=180n
M2390 t844 nw347 0 0 nch w=1u l=180n
Cnw351 nw351 0 2f
M2391 nw352 nw350 vdd vdd pch w=2u l=180n
M2392 nw352 nw351 vdd vdd pch w=2u l=180n
CT845 t845 0 0.1f
M2393 nw352 nw350 t845 0 nch w=1u l=180n
M2394 t845 nw351 0 0 nch w=1u l=180n
Cnw352 nw352 0 2f
CT846 t846 0 0.1f
CT847 t847 0 0.1f
CT848 t848 0 0.1f
M2395 t846 nw38 vdd vdd pch w=2u l=180n
M2396 t846 nw285 vdd vdd pch w=2u l=180n
CT849 t849 0 0.1f
M2397 t846 nw38 t849 0 nch w=1u l=180n
M2398 t849 nw285 0 0 nch w=1u l=180n
M2399 t847 nw38 vdd vdd pch w=2u l=180n
M2400 t847 t846 vdd vdd pch w=2u l=180n
CT850 t850 0 0.1f
M2401 t847 nw38 t850 0 nch w=1u l=180n
M2402 t850 t846 0 0 nch w=1u l=180n
M2403 t848 nw285 vdd vdd pch w=2u l=180n
M2404 t848 t846 vdd vdd pch w=2u l=180n
CT851 t851 0 0.1f
M2405 t848 nw285 t851 0 nch w=1u l=180n
M2406 t851 t846 0 0 nch w=1u l=180n
M2407 nw353 t847 vdd vdd pch w=2u l=180n
M2408 nw353 t848 vdd vdd pch w=2u l=180n
CT852 t852 0 0.1f
M2409 nw353 t847 t852 0 nch w=1u l=180n
M2410 t852 t848 0 0 nch w=1u l=180n
Cnw353 nw353 0 2f
CT853 t853 0 0.1f
CT854 t854 0 0.1f
CT855 t855 0 0.1f
M2411 t853 nw353 vdd vdd pch w=2u l=180n
M2412 t853 nw352 vdd vdd pch w=2u l=180n
CT856 t856 0 0.1f
M2413 t853 nw353 t856 0 nch w=1u l=180n
M2414 t856 nw352 0 0 nch w=1u l=180n
M2415 t854 nw353 vdd vdd pch w=2u l=180n
M2416 t854 t853 vdd vdd pch w=2u l=180n
CT857 t857 0 0.1f
M2417 t854 nw353 t857 0 nch w=1u l=180n
M2418 t857 t853 0 0 nch w=1u l=180n
M2419 t855 nw352 vdd vdd pch w=2u l=180n
M2420 t855 t853 vdd vdd pch w=2u l=180n
CT858 t858 0 0.1f
M2421 t855 nw352 t858 0 nch w=1u l=180n
M2422 t858 t853 0 0 nch w=1u l=180n
M2423 nw354 t854 vdd vdd pch w=2u l=180n
M2424 nw354 t855 vdd vdd pch w=2u l=180n
CT859 t859 0 0.1f
M2425 nw354 t854 t859 0 nch w=1u l=180n
M2426 t859 t855 0 0 nch w=1u l=180n
Cnw354 nw354 0 2f
M2427 nw355 nw38 vdd vdd pch w=2u l=180n
M2428 nw355 nw285 vdd vdd pch w=2u l=180n
CT860 t860 0 0.1f
M2429 nw355 nw38 t860 0 nch w=1u l=180n
M2430 t860 nw285 0 0 nch w=1u l=180n
Cnw355 nw355 0 2f
M2431 nw356 nw353 vdd vdd pch w=2u l=180n
M2432 nw356 nw352 vdd vdd pch w=2u l=180n
CT861 t861 0 0.1f
M2433 nw356 nw353 t861 0 nch w=1u l=180n
M2434 t861 nw352 0 0 nch w=1u l=180n
Cnw356 nw356 0 2f
M2435 nw357 nw355 vdd vdd pch w=2u l=180n
M2436 nw357 nw356 vdd vdd pch w=2u l=180n
CT862 t862 0 0.1f
M2437 nw357 nw355 t862 0 nch w=1u l=180n
M2438 t862 nw356 0 0 nch w=1u l=180n
Cnw357 nw357 0 2f
CT863 t863 0 0.1f
CT864 t864 0 0.1f
CT865 t865 0 0.1f
M2439 t863 nw39 vdd vdd pch w=2u l=180n
M2440 t863 nw290 vdd vdd pch w=2u l=180n
CT866 t866 0 0.1f
M2441 t863 nw39 t866 0 nch w=1u l=180n
M2442 t866 nw290 0 0 nch w=1u l=180n
M2443 t864 nw39 vdd vdd pch w=2u l=180n
M2444 t864 t863 vdd vdd pch w=2u l=180n
CT867 t867 0 0.1f
M2445 t864 nw39 t867 0 nch w=1u l=180n
M2446 t867 t863 0 0 nch w=1u l=180n
M2447 t865 nw290 vdd vdd pch w=2u l=180n
M2448 t865 t863 vdd vdd pch w=2u l=180n
CT868 t868 0 0.1f
M2449 t865 nw290 t868 0 nch w=1u l=180n
M2450 t868 t863 0 0 nch w=1u l=180n
M2451 nw358 t864 vdd vdd pch w=2u l=180n
M2452 nw358 t865 vdd vdd pch w=2u l=180n
CT869 t869 0 0.1f
M2453 nw358 t864 t869 0 nch w=1u l=180n
M2454 t869 t865 0 0 nch w=1u l=180n
Cnw358 nw358 0 2f
CT870 t870 0 0.1f
CT871 t871 0 0.1f
CT872 t872 0 0.1f
M2455 t870 nw358 vdd vdd pch w=2u l=180n
M2456 t870 nw357 vdd vdd pch w=2u l=180n
CT873 t873 0 0.1f
M2457 t870 nw358 t873 0 nch w=1u l=180n
M2458 t873 nw357 0 0 nch w=1u l=180n
M2459 t871 nw358 vdd vdd pch w=2u l=180n
M2460 t871 t870 vdd vdd pch w=2u l=180n
CT874 t874 0 0.1f
M2461 t871 nw358 t874 0 nch w=1u l=180n
M2462 t874 t870 0 0 nch w=1u l=180n
M2463 t872 nw357 vdd vdd pch w=2u l=180n
M2464 t872 t870 vdd vdd pch w=2u l=180n
CT875 t875 0 0.1f
M2465 t872 nw357 t875 0 nch w=1u l=180n
M2466 t875 t870 0 0 nch w=1u l=180n
M2467 nw359 t871 vdd vdd pch w=2u l=180n
M2468 nw359 t872 vdd vdd pch w=2u l=180n
CT876 t876 0 0.1f
M2469 nw359 t871 t876 0 nch w=1u l=180n
M2470 t876 t872 0 0 nch w=1u l=180n
Cnw359 nw359 0 2f
M2471 nw360 nw39 vdd vdd pch w=2u l=180n
M2472 nw360 nw290 vdd vdd pch w=2u l=180n
CT877 t877 0 0.1f
M2473 nw360 nw39 t877 0 nch w=1u l=180n
M2474 t877 nw290 0 0 nch w=1u l=180n
Cnw360 nw360 0 2f
M2475 nw361 nw358 vdd vdd pch w=2u l=180n
M2476 nw361 nw357 vdd vdd pch w=2u l=180n
CT878 t878 0 0.1f
M2477 nw361 nw358 t878 0 nch w=1u l=180n
M2478 t878 nw357 0 0 nch w=1u l=180n
Cnw361 nw361 0 2f
M2479 nw362 nw360 vdd vdd pch w=2u l=180n
M2480 nw362 nw361 vdd vdd pch w=2u l=180n
CT879 t879 0 0.1f
M2481 nw362 nw360 t879 0 nch w=1u l=180n
M2482 t879 nw361 0 0 nch w=1u l=180n
Cnw362 nw362 0 2f
CT880 t880 0 0.1f
CT881 t881 0 0.1f
CT882 t882 0 0.1f
M2483 t880 nw40 vdd vdd pch w=2u l=180n
M2484 t880 nw295 vdd vdd pch w=2u l=180n
CT883 t883 0 0.1f
M2485 t880 nw40 t883 0 nch w=1u l=180n
M2486 t883 nw295 0 0 nch w=1u l=180n
M2487 t881 nw40 vdd vdd pch w=2u l=180n
M2488 t881 t880 vdd vdd pch w=2u l=180n
CT884 t884 0 0.1f
M2489 t881 nw40 t884 0 nch w=1u l=180n
M2490 t884 t880 0 0 nch w=1u l=180n
M2491 t882 nw295 vdd vdd pch w=2u l=180n
M2492 t882 t880 vdd vdd pch w=2u l=180n
CT885 t885 0 0.1f
M2493 t882 nw295 t885 0 nch w=1u l=180n
M2494 t885 t880 0 0 nch w=1u l=180n
M2495 nw363 t881 vdd vdd pch w=2u l=180n
M2496 nw363 t882 vdd vdd pch w=2u l=180n
CT886 t886 0 0.1f
M2497 nw363 t881 t886 0 nch w=1u l=180n
M2498 t886 t882 0 0 nch w=1u l=180n
Cnw363 nw363 0 2f
CT887 t887 0 0.1f
CT888 t888 0 0.1f
CT889 t889 0 0.1f
M2499 t887 nw363 vdd vdd pch w=2u l=180n
M2500 t887 nw362 vdd vdd pch w=2u l=180n
CT890 t890 0 0.1f
M2501 t887 nw363 t890 0 nch w=1u l=180n
M2502 t890 nw362 0 0 nch w=1u l=180n
M2503 t888 nw363 vdd vdd pch w=2u l=180n
M2504 t888 t887 vdd vdd pch w=2u l=180n
CT891 t891 0 0.1f
M2505 t888 nw363 t891 0 nch w=1u l=180n
M2506 t891 t887 0 0 nch w=1u l=180n
M2507 t889 nw362 vdd vdd pch w=2u l=180n
M2508 t889 t887 vdd vdd pch w=2u l=180n
CT892 t892 0 0.1f
M2509 t889 nw362 t892 0 nch w=1u l=180n
M2510 t892 t887 0 0 nch w=1u l=180n
M2511 nw364 t888 vdd vdd pch w=2u l=180n
M2512 nw364 t889 vdd vdd pch w=2u l=180n
CT893 t893 0 0.1f
M2513 nw364 t888 t893 0 nch w=1u l=180n
M2514 t893 t889 0 0 nch w=1u l=180n
Cnw364 nw364 0 2f
M2515 nw365 nw40 vdd vdd pch w=2u l=180n
M2516 nw365 nw295 vdd vdd pch w=2u l=180n
CT894 t894 0 0.1f
M2517 nw365 nw40 t894 0 nch w=1u l=180n
M2518 t894 nw295 0 0 nch w=1u l=180n
Cnw365 nw365 0 2f
M2519 nw366 nw363 vdd vdd pch w=2u l=180n
M2520 nw366 nw362 vdd vdd pch w=2u l=180n
CT895 t895 0 0.1f
M2521 nw366 nw363 t895 0 nch w=1u l=180n
M2522 t895 nw362 0 0 nch w=1u l=180n
Cnw366 nw366 0 2f
M2523 nw367 nw365 vdd vdd pch w=2u l=180n
M2524 nw367 nw366 vdd vdd pch w=2u l=180n
CT896 t896 0 0.1f
M2525 nw367 nw365 t896 0 nch w=1u l=180n
M2526 t896 nw366 0 0 nch w=1u l=180n
Cnw367 nw367 0 2f
CT897 t897 0 0.1f
CT898 t898 0 0.1f
CT899 t899 0 0.1f
M2527 t897 nw41 vdd vdd pch w=2u l=180n
M2528 t897 nw300 vdd vdd pch w=2u l=180n
CT900 t900 0 0.1f
M2529 t897 nw41 t900 0 nch w=1u l=180n
M2530 t900 nw300 0 0 nch w=1u l=180n
M2531 t898 nw41 vdd vdd pch w=2u l=180n
M2532 t898 t897 vdd vdd pch w=2u l=180n
CT901 t901 0 0.1f
M2533 t898 nw41 t901 0 nch w=1u l=180n
M2534 t901 t897 0 0 nch w=1u l=180n
M2535 t899 nw300 vdd vdd pch w=2u l=180n
M2536 t899 t897 vdd vdd pch w=2u l=180n
CT902 t902 0 0.1f
M2537 t899 nw300 t902 0 nch w=1u l=180n
M2538 t902 t897 0 0 nch w=1u l=180n
M2539 nw368 t898 vdd vdd pch w=2u l=180n
M2540 nw368 t899 vdd vdd pch w=2u l=180n
CT903 t903 0 0.1f
M2541 nw368 t898 t903 0 nch w=1u l=180n
M2542 t903 t899 0 0 nch w=1u l=180n
Cnw368 nw368 0 2f
CT904 t904 0 0.1f
CT905 t905 0 0.1f
CT906 t906 0 0.1f
M2543 t904 nw368 vdd vdd pch w=2u l=180n
M2544 t904 nw367 vdd vdd pch w=2u l=180n
CT907 t907 0 0.1f
M2545 t904 nw368 t907 0 nch w=1u l=180n
M2546 t907 nw367 0 0 nch w=1u l=180n
M2547 t905 nw368 vdd vdd pch w=2u l=180n
M2548 t905 t904 vdd vdd pch w=2u l=180n
CT908 t908 0 0.1f
M2549 t905 nw368 t908 0 nch w=1u l=180n
M2550 t908 t904 0 0 nch w=1u l=180n
M2551 t906 nw367 vdd vdd pch w=2u l=180n
M2552 t906 t904 vdd vdd pch w=2u l=180n
CT909 t909 0 0.1f
M2553 t906 nw367 t909 0 nch w=1u l=180n
M2554 t909 t904 0 0 nch w=1u l=180n
M2555 nw369 t905 vdd vdd pch w=2u l=180n
M2556 nw369 t906 vdd vdd pch w=2u l=180n
CT910 t910 0 0.1f
M2557 nw369 t905 t910 0 nch w=1u l=180n
M2558 t910 t906 0 0 nch w=1u l=180n
Cnw369 nw369 0 2f
M2559 nw370 nw41 vdd vdd pch w=2u l=180n
M2560 nw370 nw300 vdd vdd pch w=2u l=180n
CT911 t911 0 0.1f
M2561 nw370 nw41 t911 0 nch w=1u l=180n
M2562 t911 nw300 0 0 nch w=1u l=180n
Cnw370 nw370 0 2f
M2563 nw371 nw368 vdd vdd pch w=2u l=180n
M2564 nw371 nw367 vdd vdd pch w=2u l=180n
CT912 t912 0 0.1f
M2565 nw371 nw368 t912 0 nch w=1u l=180n
M2566 t912 nw367 0 0 nch w=1u l=180n
Cnw371 nw371 0 2f
M2567 nw372 nw370 vdd vdd pch w=2u l=180n
M2568 nw372 nw371 vdd vdd pch w=2u l=180n
CT913 t913 0 0.1f
M2569 nw372 nw370 t913 0 nch w=1u l=180n
M2570 t913 nw371 0 0 nch w=1u l=180n
Cnw372 nw372 0 2f
CT914 t914 0 0.1f
CT915 t915 0 0.1f
CT916 t916 0 0.1f
M2571 t914 nw42 vdd vdd pch w=2u l=180n
M2572 t914 nw305 vdd vdd pch w=2u l=180n
CT917 t917 0 0.1f
M2573 t914 nw42 t917 0 nch w=1u l=180n
M2574 t917 nw305 0 0 nch w=1u l=180n
M2575 t915 nw42 vdd vdd pch w=2u l=180n
M2576 t915 t914 vdd vdd pch w=2u l=180n
CT918 t918 0 0.1f
M2577 t915 nw42 t918 0 nch w=1u l=180n
M2578 t918 t914 0 0 nch w=1u l=180n
M2579 t916 nw305 vdd vdd pch w=2u l=180n
M2580 t916 t914 vdd vdd pch w=2u l=180n
CT919 t919 0 0.1f
M2581 t916 nw305 t919 0 nch w=1u l=180n
M2582 t919 t914 0 0 nch w=1u l=180n
M2583 nw373 t915 vdd vdd pch w=2u l=180n
M2584 nw373 t916 vdd vdd pch w=2u l=180n
CT920 t920 0 0.1f
M2585 nw373 t915 t920 0 nch w=1u l=180n
M2586 t920 t916 0 0 nch w=1u l=180n
Cnw373 nw373 0 2f
CT921 t921 0 0.1f
CT922 t922 0 0.1f
CT923 t923 0 0.1f
M2587 t921 nw373 vdd vdd pch w=2u l=180n
M2588 t921 nw372 vdd vdd pch w=2u l=180n
CT924 t924 0 0.1f
M2589 t921 nw373 t924 0 nch w=1u l=180n
M2590 t924 nw372 0 0 nch w=1u l=180n
M2591 t922 nw373 vdd vdd pch w=2u l=180n
M2592 t922 t921 vdd vdd pch w=2u l=180n
CT925 t925 0 0.1f
M2593 t922 nw373 t925 0 nch w=1u l=180n
M2594 t925 t921 0 0 nch w=1u l=180n
M2595 t923 nw372 vdd vdd pch w=2u l=180n
M2596 t923 t921 vdd vdd pch w=2u l=180n
CT926 t926 0 0.1f
M2597 t923 nw372 t926 0 nch w=1u l=180n
M2598 t926 t921 0 0 nch w=1u l=180n
M2599 nw374 t922 vdd vdd pch w=2u l=180n
M2600 nw374 t923 vdd vdd pch w=2u l=180n
CT927 t927 0 0.1f
M2601 nw374 t922 t927 0 nch w=1u l=180n
M2602 t927 t923 0 0 nch w=1u l=180n
Cnw374 nw374 0 2f
M2603 nw375 nw42 vdd vdd pch w=2u l=180n
M2604 nw375 nw305 vdd vdd pch w=2u l=180n
CT928 t928 0 0.1f
M2605 nw375 nw42 t928 0 nch w=1u l=180n
M2606 t928 nw305 0 0 nch w=1u l=180n
Cnw375 nw375 0 2f
M2607 nw376 nw373 vdd vdd pch w=2u l=180n
M2608 nw376 nw372 vdd vdd pch w=2u l=180n
CT929 t929 0 0.1f
M2609 nw376 nw373 t929 0 nch w=1u l=180n
M2610 t929 nw372 0 0 nch w=1u l=180n
Cnw376 nw376 0 2f
M2611 nw377 nw375 vdd vdd pch w=2u l=180n
M2612 nw377 nw376 vdd vdd pch w=2u l=180n
CT930 t930 0 0.1f
M2613 nw377 nw375 t930 0 nch w=1u l=180n
M2614 t930 nw376 0 0 nch w=1u l=180n
Cnw377 nw377 0 2f
CT931 t931 0 0.1f
CT932 t932 0 0.1f
CT933 t933 0 0.1f
M2615 t931 nw43 vdd vdd pch w=2u l=180n
M2616 t931 nw310 vdd vdd pch w=2u l=180n
CT934 t934 0 0.1f
M2617 t931 nw43 t934 0 nch w=1u l=180n
M2618 t934 nw310 0 0 nch w=1u l=180n
M2619 t932 nw43 vdd vdd pch w=2u l=180n
M2620 t932 t931 vdd vdd pch w=2u l=180n
CT935 t935 0 0.1f
M2621 t932 nw43 t935 0 nch w=1u l=180n
M2622 t935 t931 0 0 nch w=1u l=180n
M2623 t933 nw310 vdd vdd pch w=2u l=180n
M2624 t933 t931 vdd vdd pch w=2u l=180n
CT936 t936 0 0.1f
M2625 t933 nw310 t936 0 nch w=1u l=180n
M2626 t936 t931 0 0 nch w=1u l=180n
M2627 nw378 t932 vdd vdd pch w=2u l=180n
M2628 nw378 t933 vdd vdd pch w=2u l=180n
CT937 t937 0 0.1f
M2629 nw378 t932 t937 0 nch w=1u l=180n
M2630 t937 t933 0 0 nch w=1u l=180n
Cnw378 nw378 0 2f
CT938 t938 0 0.1f
CT939 t939 0 0.1f
CT940 t940 0 0.1f
M2631 t938 nw378 vdd vdd pch w=2u l=180n
M2632 t938 nw377 vdd vdd pch w=2u l=180n
CT941 t941 0 0.1f
M2633 t938 nw378 t941 0 nch w=1u l=180n
M2634 t941 nw377 0 0 nch w=1u l=180n
M2635 t939 nw378 vdd vdd pch w=2u l=180n
M2636 t939 t938 vdd vdd pch w=2u l=180n
CT942 t942 0 0.1f
M2637 t939 nw378 t942 0 nch w=1u l=180n
M2638 t942 t938 0 0 nch w=1u l=180n
M2639 t940 nw377 vdd vdd pch w=2u l=180n
M2640 t940 t938 vdd vdd pch w=2u l=180n
CT943 t943 0 0.1f
M2641 t940 nw377 t943 0 nch w=1u l=180n
M2642 t943 t938 0 0 nch w=1u l=180n
M2643 nw379 t939 vdd vdd pch w=2u l=180n
M2644 nw379 t940 vdd vdd pch w=2u l=180n
CT944 t944 0 0.1f
M2645 nw379 t939 t944 0 nch w=1u l=180n
M2646 t944 t940 0 0 nch w=1u l=180n
Cnw379 nw379 0 2f
M2647 nw380 nw43 vdd vdd pch w=2u l=180n
M2648 nw380 nw310 vdd vdd pch w=2u l=180n
CT945 t945 0 0.1f
M2649 nw380 nw43 t945 0 nch w=1u l=180n
M2650 t945 nw310 0 0 nch w=1u l=180n
Cnw380 nw380 0 2f
M2651 nw381 nw378 vdd vdd pch w=2u l=180n
M2652 nw381 nw377 vdd vdd pch w=2u l=180n
CT946 t946 0 0.1f
M2653 nw381 nw378 t946 0 nch w=1u l=180n
M2654 t946 nw377 0 0 nch w=1u l=180n
Cnw381 nw381 0 2f
M2655 nw382 nw380 vdd vdd pch w=2u l=180n
M2656 nw382 nw381 vdd vdd pch w=2u l=180n
CT947 t947 0 0.1f
M2657 nw382 nw380 t947 0 nch w=1u l=180n
M2658 t947 nw381 0 0 nch w=1u l=180n
Cnw382 nw382 0 2f
CT948 t948 0 0.1f
CT949 t949 0 0.1f
CT950 t950 0 0.1f
M2659 t948 nw44 vdd vdd pch w=2u l=180n
M2660 t948 nw315 vdd vdd pch w=2u l=180n
CT951 t951 0 0.1f
M2661 t948 nw44 t951 0 nch w=1u l=180n
M2662 t951 nw315 0 0 nch w=1u l=180n
M2663 t949 nw44 vdd vdd pch w=2u l=180n
M2664 t949 t948 vdd vdd pch w=2u l=180n
CT952 t952 0 0.1f
M2665 t949 nw44 t952 0 nch w=1u l=180n
M2666 t952 t948 0 0 nch w=1u l=180n
M2667 t950 nw315 vdd vdd pch w=2u l=180n
M2668 t950 t948 vdd vdd pch w=2u l=180n
CT953 t953 0 0.1f
M2669 t950 nw315 t953 0 nch w=1u l=180n
M2670 t953 t948 0 0 nch w=1u l=180n
M2671 nw383 t949 vdd vdd pch w=2u l=180n
M2672 nw383 t950 vdd vdd pch w=2u l=180n
CT954 t954 0 0.1f
M2673 nw383 t949 t954 0 nch w=1u l=180n
M2674 t954 t950 0 0 nch w=1u l=180n
Cnw383 nw383 0 2f
CT955 t955 0 0.1f
CT956 t956 0 0.1f
CT957 t957 0 0.1f
M2675 t955 nw383 vdd vdd pch w=2u l=180n
M2676 t955 nw382 vdd vdd pch w=2u l=180n
CT958 t958 0 0.1f
M2677 t955 nw383 t958 0 nch w=1u l=180n
M2678 t958 nw382 0 0 nch w=1u l=180n
M2679 t956 nw383 vdd vdd pch w=2u l=180n
M2680 t956 t955 vdd vdd pch w=2u l=180n
CT959 t959 0 0.1f
M2681 t956 nw383 t959 0 nch w=1u l=180n
M2682 t959 t955 0 0 nch w=1u l=180n
M2683 t957 nw382 vdd vdd pch w=2u l=180n
M2684 t957 t955 vdd vdd pch w=2u l=180n
CT960 t960 0 0.1f
M2685 t957 nw382 t960 0 nch w=1u l=180n
M2686 t960 t955 0 0 nch w=1u l=180n
M2687 nw384 t956 vdd vdd pch w=2u l=180n
M2688 nw384 t957 vdd vdd pch w=2u l=180n
CT961 t961 0 0.1f
M2689 nw384 t956 t961 0 nch w=1u l=180n
M2690 t961 t957 0 0 nch w=1u l=180n
Cnw384 nw384 0 2f
M2691 nw385 nw44 vdd vdd pch w=2u l=180n
M2692 nw385 nw315 vdd vdd pch w=2u l=180n
CT962 t962 0 0.1f
M2693 nw385 nw44 t962 0 nch w=1u l=180n
M2694 t962 nw315 0 0 nch w=1u l=180n
Cnw385 nw385 0 2f
M2695 nw386 nw383 vdd vdd pch w=2u l=180n
M2696 nw386 nw382 vdd vdd pch w=2u l=180n
CT963 t963 0 0.1f
M2697 nw386 nw383 t963 0 nch w=1u l=180n
M2698 t963 nw382 0 0 nch w=1u l=180n
Cnw386 nw386 0 2f
M2699 nw387 nw385 vdd vdd pch w=2u l=180n
M2700 nw387 nw386 vdd vdd pch w=2u l=180n
CT964 t964 0 0.1f
M2701 nw387 nw385 t964 0 nch w=1u l=180n
M2702 t964 nw386 0 0 nch w=1u l=180n
Cnw387 nw387 0 2f
CT965 t965 0 0.1f
CT966 t966 0 0.1f
CT967 t967 0 0.1f
M2703 t965 nw45 vdd vdd pch w=2u l=180n
M2704 t965 nw320 vdd vdd pch w=2u l=180n
CT968 t968 0 0.1f
M2705 t965 nw45 t968 0 nch w=1u l=180n
M2706 t968 nw320 0 0 nch w=1u l=180n
M2707 t966 nw45 vdd vdd pch w=2u l=180n
M2708 t966 t965 vdd vdd pch w=2u l=180n
CT969 t969 0 0.1f
M2709 t966 nw45 t969 0 nch w=1u l=180n
M2710 t969 t965 0 0 nch w=1u l=180n
M2711 t967 nw320 vdd vdd pch w=2u l=180n
M2712 t967 t965 vdd vdd pch w=2u l=180n
CT970 t970 0 0.1f
M2713 t967 nw320 t970 0 nch w=1u l=180n
M2714 t970 t965 0 0 nch w=1u l=180n
M2715 nw388 t966 vdd vdd pch w=2u l=180n
M2716 nw388 t967 vdd vdd pch w=2u l=180n
CT971 t971 0 0.1f
M2717 nw388 t966 t971 0 nch w=1u l=180n
M2718 t971 t967 0 0 nch w=1u l=180n
Cnw388 nw388 0 2f
CT972 t972 0 0.1f
CT973 t973 0 0.1f
CT974 t974 0 0.1f
M2719 t972 nw388 vdd vdd pch w=2u l=180n
M2720 t972 nw387 vdd vdd pch w=2u l=180n
CT975 t975 0 0.1f
M2721 t972 nw388 t975 0 nch w=1u l=180n
M2722 t975 nw387 0 0 nch w=1u l=180n
M2723 t973 nw388 vdd vdd pch w=2u l=180n
M2724 t973 t972 vdd vdd pch w=2u l=180n
CT976 t976 0 0.1f
M2725 t973 nw388 t976 0 nch w=1u l=180n
M2726 t976 t972 0 0 nch w=1u l=180n
M2727 t974 nw387 vdd vdd pch w=2u l=180n
M2728 t974 t972 vdd vdd pch w=2u l=180n
CT977 t977 0 0.1f
M2729 t974 nw387 t977 0 nch w=1u l=180n
M2730 t977 t972 0 0 nch w=1u l=180n
M2731 nw389 t973 vdd vdd pch w=2u l=180n
M2732 nw389 t974 vdd vdd pch w=2u l=180n
CT978 t978 0 0.1f
M2733 nw389 t973 t978 0 nch w=1u l=180n
M2734 t978 t974 0 0 nch w=1u l=180n
Cnw389 nw389 0 2f
M2735 nw390 nw45 vdd vdd pch w=2u l=180n
M2736 nw390 nw320 vdd vdd pch w=2u l=180n
CT979 t979 0 0.1f
M2737 nw390 nw45 t979 0 nch w=1u l=180n
M2738 t979 nw320 0 0 nch w=1u l=180n
Cnw390 nw390 0 2f
M2739 nw391 nw388 vdd vdd pch w=2u l=180n
M2740 nw391 nw387 vdd vdd pch w=2u l=180n
CT980 t980 0 0.1f
M2741 nw391 nw388 t980 0 nch w=1u l=180n
M2742 t980 nw387 0 0 nch w=1u l=180n
Cnw391 nw391 0 2f
M2743 nw392 nw390 vdd vdd pch w=2u l=180n
M2744 nw392 nw391 vdd vdd pch w=2u l=180n
CT981 t981 0 0.1f
M2745 nw392 nw390 t981 0 nch w=1u l=180n
M2746 t981 nw391 0 0 nch w=1u l=180n
Cnw392 nw392 0 2f
CT982 t982 0 0.1f
CT983 t983 0 0.1f
CT984 t984 0 0.1f
M2747 t982 nw46 vdd vdd pch w=2u l=180n
M2748 t982 nw325 vdd vdd pch w=2u l=180n
CT985 t985 0 0.1f
M2749 t982 nw46 t985 0 nch w=1u l=180n
M2750 t985 nw325 0 0 nch w=1u l=180n
M2751 t983 nw46 vdd vdd pch w=2u l=180n
M2752 t983 t982 vdd vdd pch w=2u l=180n
CT986 t986 0 0.1f
M2753 t983 nw46 t986 0 nch w=1u l=180n
M2754 t986 t982 0 0 nch w=1u l=180n
M2755 t984 nw325 vdd vdd pch w=2u l=180n
M2756 t984 t982 vdd vdd pch w=2u l=180n
CT987 t987 0 0.1f
M2757 t984 nw325 t987 0 nch w=1u l=180n
M2758 t987 t982 0 0 nch w=1u l=180n
M2759 nw393 t983 vdd vdd pch w=2u l=180n
M2760 nw393 t984 vdd vdd pch w=2u l=180n
CT988 t988 0 0.1f
M2761 nw393 t983 t988 0 nch w=1u l=180n
M2762 t988 t984 0 0 nch w=1u l=180n
Cnw393 nw393 0 2f
CT989 t989 0 0.1f
CT990 t990 0 0.1f
CT991 t991 0 0.1f
M2763 t989 nw393 vdd vdd pch w=2u l=180n
M2764 t989 nw392 vdd vdd pch w=2u l=180n
CT992 t992 0 0.1f
M2765 t989 nw393 t992 0 nch w=1u l=180n
M2766 t992 nw392 0 0 nch w=1u l=180n
M2767 t990 nw393 vdd vdd pch w=2u l=180n
M2768 t990 t989 vdd vdd pch w=2u l=180n
CT993 t993 0 0.1f
M2769 t990 nw393 t993 0 nch w=1u l=180n
M2770 t993 t989 0 0 nch w=1u l=180n
M2771 t991 nw392 vdd vdd pch w=2u l=180n
M2772 t991 t989 vdd vdd pch w=2u l=180n
CT994 t994 0 0.1f
M2773 t991 nw392 t994 0 nch w=1u l=180n
M2774 t994 t989 0 0 nch w=1u l=180n
M2775 nw394 t990 vdd vdd pch w=2u l=180n
M2776 nw394 t991 vdd vdd pch w=2u l=180n
CT995 t995 0 0.1f
M2777 nw394 t990 t995 0 nch w=1u l=180n
M2778 t995 t991 0 0 nch w=1u l=180n
Cnw394 nw394 0 2f
M2779 nw395 nw46 vdd vdd pch w=2u l=180n
M2780 nw395 nw325 vdd vdd pch w=2u l=180n
CT996 t996 0 0.1f
M2781 nw395 nw46 t996 0 nch w=1u l=180n
M2782 t996 nw325 0 0 nch w=1u l=180n
Cnw395 nw395 0 2f
M2783 nw396 nw393 vdd vdd pch w=2u l=180n
M2784 nw396 nw392 vdd vdd pch w=2u l=180n
CT997 t997 0 0.1f
M2785 nw396 nw393 t997 0 nch w=1u l=180n
M2786 t997 nw392 0 0 nch w=1u l=180n
Cnw396 nw396 0 2f
M2787 nw397 nw395 vdd vdd pch w=2u l=180n
M2788 nw397 nw396 vdd vdd pch w=2u l=180n
CT998 t998 0 0.1f
M2789 nw397 nw395 t998 0 nch w=1u l=180n
M2790 t998 nw396 0 0 nch w=1u l=180n
Cnw397 nw397 0 2f
CT999 t999 0 0.1f
CT1000 t1000 0 0.1f
CT1001 t1001 0 0.1f
M2791 t999 nw47 vdd vdd pch w=2u l=180n
M2792 t999 nw329 vdd vdd pch w=2u l=180n
CT1002 t1002 0 0.1f
M2793 t999 nw47 t1002 0 nch w=1u l=180n
M2794 t1002 nw329 0 0 nch w=1u l=180n
M2795 t1000 nw47 vdd vdd pch w=2u l=180n
M2796 t1000 t999 vdd vdd pch w=2u l=180n
CT1003 t1003 0 0.1f
M2797 t1000 nw47 t1003 0 nch w=1u l=180n
M2798 t1003 t999 0 0 nch w=1u l=180n
M2799 t1001 nw329 vdd vdd pch w=2u l=180n
M2800 t1001 t999 vdd vdd pch w=2u l=180n
CT1004 t1004 0 0.1f
M2801 t1001 nw329 t1004 0 nch w=1u l=180n
M2802 t1004 t999 0 0 nch w=1u l=180n
M2803 nw398 t1000 vdd vdd pch w=2u l=180n
M2804 nw398 t1001 vdd vdd pch w=2u l=180n
CT1005 t1005 0 0.1f
M2805 nw398 t1000 t1005 0 nch w=1u l=180n
M2806 t1005 t1001 0 0 nch w=1u l=180n
Cnw398 nw398 0 2f
CT1006 t1006 0 0.1f
CT1007 t1007 0 0.1f
CT1008 t1008 0 0.1f
M2807 t1006 nw398 vdd vdd pch w=2u l=180n
M2808 t1006 nw397 vdd vdd pch w=2u l=180n
CT1009 t1009 0 0.1f
M2809 t1006 nw398 t1009 0 nch w=1u l=180n
M2810 t1009 nw397 0 0 nch w=1u l=180n
M2811 t1007 nw398 vdd vdd pch w=2u l=180n
M2812 t1007 t1006 vdd vdd pch w=2u l=180n
CT1010 t1010 0 0.1f
M2813 t1007 nw398 t1010 0 nch w=1u l=180n
M2814 t1010 t1006 0 0 nch w=1u l=180n
M2815 t1008 nw397 vdd vdd pch w=2u l=180n
M2816 t1008 t1006 vdd vdd pch w=2u l=180n
CT1011 t1011 0 0.1f
M2817 t1008 nw397 t1011 0 nch w=1u l=180n
M2818 t1011 t1006 0 0 nch w=1u l=180n
M2819 nw399 t1007 vdd vdd pch w=2u l=180n
M2820 nw399 t1008 vdd vdd pch w=2u l=180n
CT1012 t1012 0 0.1f
M2821 nw399 t1007 t1012 0 nch w=1u l=180n
M2822 t1012 t1008 0 0 nch w=1u l=180n
Cnw399 nw399 0 2f
M2823 nw400 nw47 vdd vdd pch w=2u l=180n
M2824 nw400 nw329 vdd vdd pch w=2u l=180n
CT1013 t1013 0 0.1f
M2825 nw400 nw47 t1013 0 nch w=1u l=180n
M2826 t1013 nw329 0 0 nch w=1u l=180n
Cnw400 nw400 0 2f
M2827 nw401 nw398 vdd vdd pch w=2u l=180n
M2828 nw401 nw397 vdd vdd pch w=2u l=180n
CT1014 t1014 0 0.1f
M2829 nw401 nw398 t1014 0 nch w=1u l=180n
M2830 t1014 nw397 0 0 nch w=1u l=180n
Cnw401 nw401 0 2f
M2831 nw402 nw400 vdd vdd pch w=2u l=180n
M2832 nw402 nw401 vdd vdd pch w=2u l=180n
CT1015 t1015 0 0.1f
M2833 nw402 nw400 t1015 0 nch w=1u l=180n
M2834 t1015 nw401 0 0 nch w=1u l=180n
Cnw402 nw402 0 2f
CT1016 t1016 0 0.1f
CT1017 t1017 0 0.1f
CT1018 t1018 0 0.1f
M2835 t1016 nw48 vdd vdd pch w=2u l=180n
M2836 t1016 nw330 vdd vdd pch w=2u l=180n
CT1019 t1019 0 0.1f
M2837 t1016 nw48 t1019 0 nch w=1u l=180n
M2838 t1019 nw330 0 0 nch w=1u l=180n
M2839 t1017 nw48 vdd vdd pch w=2u l=180n
M2840 t1017 t1016 vdd vdd pch w=2u l=180n
CT1020 t1020 0 0.1f
M2841 t1017 nw48 t1020 0 nch w=1u l=180n
M2842 t1020 t1016 0 0 nch w=1u l=180n
M2843 t1018 nw330 vdd vdd pch w=2u l=180n
M2844 t1018 t1016 vdd vdd pch w=2u l=180n
CT1021 t1021 0 0.1f
M2845 t1018 nw330 t1021 0 nch w=1u l=180n
M2846 t1021 t1016 0 0 nch w=1u l=180n
M2847 nw403 t1017 vdd vdd pch w=2u l=180n
M2848 nw403 t1018 vdd vdd pch w=2u l=180n
CT1022 t1022 0 0.1f
M2849 nw403 t1017 t1022 0 nch w=1u l=180n
M2850 t1022 t1018 0 0 nch w=1u l=180n
Cnw403 nw403 0 2f
CT1023 t1023 0 0.1f
CT1024 t1024 0 0.1f
CT1025 t1025 0 0.1f
M2851 t1023 nw403 vdd vdd pch w=2u l=180n
M2852 t1023 nw402 vdd vdd pch w=2u l=180n
CT1026 t1026 0 0.1f
M2853 t1023 nw403 t1026 0 nch w=1u l=180n
M2854 t1026 nw402 0 0 nch w=1u l=180n
M2855 t1024 nw403 vdd vdd pch w=2u l=180n
M2856 t1024 t1023 vdd vdd pch w=2u l=180n
CT1027 t1027 0 0.1f
M2857 t1024 nw403 t1027 0 nch w=1u l=180n
M2858 t1027 t1023 0 0 nch w=1u l=180n
M2859 t1025 nw402 vdd vdd pch w=2u l=180n
M2860 t1025 t1023 vdd vdd pch w=2u l=180n
CT1028 t1028 0 0.1f
M2861 t1025 nw402 t1028 0 nch w=1u l=180n
M2862 t1028 t1023 0 0 nch w=1u l=180n
M2863 nw404 t1024 vdd vdd pch w=2u l=180n
M2864 nw404 t1025 vdd vdd pch w=2u l=180n
CT1029 t1029 0 0.1f
M2865 nw404 t1024 t1029 0 nch w=1u l=180n
M2866 t1029 t1025 0 0 nch w=1u l=180n
Cnw404 nw404 0 2f
M2867 nw405 nw48 vdd vdd pch w=2u l=180n
M2868 nw405 nw330 vdd vdd pch w=2u l=180n
CT1030 t1030 0 0.1f
M2869 nw405 nw48 t1030 0 nch w=1u l=180n
M2870 t1030 nw330 0 0 nch w=1u l=180n
Cnw405 nw405 0 2f
M2871 nw406 nw403 vdd vdd pch w=2u l=180n
M2872 nw406 nw402 vdd vdd pch w=2u l=180n
CT1031 t1031 0 0.1f
M2873 nw406 nw403 t1031 0 nch w=1u l=180n
M2874 t1031 nw402 0 0 nch w=1u l=180n
Cnw406 nw406 0 2f
M2875 nw407 nw405 vdd vdd pch w=2u l=180n
M2876 nw407 nw406 vdd vdd pch w=2u l=180n
CT1032 t1032 0 0.1f
M2877 nw407 nw405 t1032 0 nch w=1u l=180n
M2878 t1032 nw406 0 0 nch w=1u l=180n
Cnw407 nw407 0 2f
CT1033 t1033 0 0.1f
CT1034 t1034 0 0.1f
CT1035 t1035 0 0.1f
M2879 t1033 nw49 vdd vdd pch w=2u l=180n
M2880 t1033 nw334 vdd vdd pch w=2u l=180n
CT1036 t1036 0 0.1f
M2881 t1033 nw49 t1036 0 nch w=1u l=180n
M2882 t1036 nw334 0 0 nch w=1u l=180n
M2883 t1034 nw49 vdd vdd pch w=2u l=180n
M2884 t1034 t1033 vdd vdd pch w=2u l=180n
CT1037 t1037 0 0.1f
M2885 t1034 nw49 t1037 0 nch w=1u l=180n
M2886 t1037 t1033 0 0 nch w=1u l=180n
M2887 t1035 nw334 vdd vdd pch w=2u l=180n
M2888 t1035 t1033 vdd vdd pch w=2u l=180n
CT1038 t1038 0 0.1f
M2889 t1035 nw334 t1038 0 nch w=1u l=180n
M2890 t1038 t1033 0 0 nch w=1u l=180n
M2891 nw408 t1034 vdd vdd pch w=2u l=180n
M2892 nw408 t1035 vdd vdd pch w=2u l=180n
CT1039 t1039 0 0.1f
M2893 nw408 t1034 t1039 0 nch w=1u l=180n
M2894 t1039 t1035 0 0 nch w=1u l=180n
Cnw408 nw408 0 2f
CT1040 t1040 0 0.1f
M2895 t1040 nw49 vdd vdd pch w=2u l=180n
M2896 t1040 nw334 vdd vdd pch w=2u l=180n
CT1041 t1041 0 0.1f
M2897 t1040 nw49 t1041 0 nch w=1u l=180n
M2898 t1041 nw334 0 0 nch w=1u l=180n
M2899 nw409 t1040 vdd vdd pch w=2u l=180n
M2900 nw409 t1040 0 0 nch w=1u l=180n
Cnw409 nw409 0 2f
CT1042 t1042 0 0.1f
CT1043 t1043 0 0.1f
CT1044 t1044 0 0.1f
M2901 t1042 nw50 vdd vdd pch w=2u l=180n
M2902 t1042 nw339 vdd vdd pch w=2u l=180n
CT1045 t1045 0 0.1f
M2903 t1042 nw50 t1045 0 nch w=1u l=180n
M2904 t1045 nw339 0 0 nch w=1u l=180n
M2905 t1043 nw50 vdd vdd pch w=2u l=180n
M2906 t1043 t1042 vdd vdd pch w=2u l=180n
CT1046 t1046 0 0.1f
M2907 t1043 nw50 t1046 0 nch w=1u l=180n
M2908 t1046 t1042 0 0 nch w=1u l=180n
M2909 t1044 nw339 vdd vdd pch w=2u l=180n
M2910 t1044 t1042 vdd vdd pch w=2u l=180n
CT1047 t1047 0 0.1f
M2911 t1044 nw339 t1047 0 nch w=1u l=180n
M2912 t1047 t1042 0 0 nch w=1u l=180n
M2913 nw410 t1043 vdd vdd pch w=2u l=180n
M2914 nw410 t1044 vdd vdd pch w=2u l=180n
CT1048 t1048 0 0.1f
M2915 nw410 t1043 t1048 0 nch w=1u l=180n
M2916 t1048 t1044 0 0 nch w=1u l=180n
Cnw410 nw410 0 2f
CT1049 t1049 0 0.1f
CT1050 t1050 0 0.1f
CT1051 t1051 0 0.1f
M2917 t1049 nw410 vdd vdd pch w=2u l=180n
M2918 t1049 nw409 vdd vdd pch w=2u l=180n
CT1052 t1052 0 0.1f
M2919 t1049 nw410 t1052 0 nch w=1u l=180n
M2920 t1052 nw409 0 0 nch w=1u l=180n
M2921 t1050 nw410 vdd vdd pch w=2u l=180n
M2922 t1050 t1049 vdd vdd pch w=2u l=180n
CT1053 t1053 0 0.1f
M2923 t1050 nw410 t1053 0 nch w=1u l=180n
M2924 t1053 t1049 0 0 nch w=1u l=180n
M2925 t1051 nw409 vdd vdd pch w=2u l=180n
M2926 t1051 t1049 vdd vdd pch w=2u l=180n
CT1054 t1054 0 0.1f
M2927 t1051 nw409 t1054 0 nch w=1u l=180n
M2928 t1054 t1049 0 0 nch w=1u l=180n
M2929 nw411 t1050 vdd vdd pch w=2u l=180n
M2930 nw411 t1051 vdd vdd pch w=2u l=180n
CT1055 t1055 0 0.1f
M2931 nw411 t1050 t1055 0 nch w=1u l=180n
M2932 t1055 t1051 0 0 nch w=1u l=180n
Cnw411 nw411 0 2f
M2933 nw412 nw50 vdd vdd pch w=2u l=180n
M2934 nw412 nw339 vdd vdd pch w=2u l=180n
CT1056 t1056 0 0.1f
M2935 nw412 nw50 t1056 0 nch w=1u l=180n
M2936 t1056 nw339 0 0 nch w=1u l=180n
Cnw412 nw412 0 2f
M2937 nw413 nw410 vdd vdd pch w=2u l=180n
M2938 nw413 nw409 vdd vdd pch w=2u l=180n
CT1057 t1057 0 0.1f
M2939 nw413 nw410 t1057 0 nch w=1u l=180n
M2940 t1057 nw409 0 0 nch w=1u l=180n
Cnw413 nw413 0 2f
M2941 nw414 nw412 vdd vdd pch w=2u l=180n
M2942 nw414 nw413 vdd vdd pch w=2u l=180n
CT1058 t1058 0 0.1f
M2943 nw414 nw412 t1058 0 nch w=1u l=180n
M2944 t1058 nw413 0 0 nch w=1u l=180n
Cnw414 nw414 0 2f
CT1059 t1059 0 0.1f
CT1060 t1060 0 0.1f
CT1061 t1061 0 0.1f
M2945 t1059 nw51 vdd vdd pch w=2u l=180n
M2946 t1059 nw344 vdd vdd pch w=2u l=180n
CT1062 t1062 0 0.1f
M2947 t1059 nw51 t1062 0 nch w=1u l=180n
M2948 t1062 nw344 0 0 nch w=1u l=180n
M2949 t1060 nw51 vdd vdd pch w=2u l=180n
M2950 t1060 t1059 vdd vdd pch w=2u l=180n
CT1063 t1063 0 0.1f
M2951 t1060 nw51 t1063 0 nch w=1u l=180n
M2952 t1063 t1059 0 0 nch w=1u l=180n
M2953 t1061 nw344 vdd vdd pch w=2u l=180n
M2954 t1061 t1059 vdd vdd pch w=2u l=180n
CT1064 t1064 0 0.1f
M2955 t1061 nw344 t1064 0 nch w=1u l=180n
M2956 t1064 t1059 0 0 nch w=1u l=180n
M2957 nw415 t1060 vdd vdd pch w=2u l=180n
M2958 nw415 t1061 vdd vdd pch w=2u l=180n
CT1065 t1065 0 0.1f
M2959 nw415 t1060 t1065 0 nch w=1u l=180n
M2960 t1065 t1061 0 0 nch w=1u l=180n
Cnw415 nw415 0 2f
CT1066 t1066 0 0.1f
CT1067 t1067 0 0.1f
CT1068 t1068 0 0.1f
M2961 t1066 nw415 vdd vdd pch w=2u l=180n
M2962 t1066 nw414 vdd vdd pch w=2u l=180n
CT1069 t1069 0 0.1f
M2963 t1066 nw415 t1069 0 nch w=1u l=180n
M2964 t1069 nw414 0 0 nch w=1u l=180n
M2965 t1067 nw415 vdd vdd pch w=2u l=180n
M2966 t1067 t1066 vdd vdd pch w=2u l=180n
CT1070 t1070 0 0.1f
M2967 t1067 nw415 t1070 0 nch w=1u l=180n
M2968 t1070 t1066 0 0 nch w=1u l=180n
M2969 t1068 nw414 vdd vdd pch w=2u l=180n
M2970 t1068 t1066 vdd vdd pch w=2u l=180n
CT1071 t1071 0 0.1f
M2971 t1068 nw414 t1071 0 nch w=1u l=180n
M2972 t1071 t1066 0 0 nch w=1u l=180n
M2973 nw416 t1067 vdd vdd pch w=2u l=180n
M2974 nw416 t1068 vdd vdd pch w=2u l=180n
CT1072 t1072 0 0.1f
M2975 nw416 t1067 t1072 0 nch w=1u l=180n
M2976 t1072 t1068 0 0 nch w=1u l=180n
Cnw416 nw416 0 2f
M2977 nw417 nw51 vdd vdd pch w=2u l=180n
M2978 nw417 nw344 vdd vdd pch w=2u l=180n
CT1073 t1073 0 0.1f
M2979 nw417 nw51 t1073 0 nch w=1u l=180n
M2980 t1073 nw344 0 0 nch w=1u l=180n
Cnw417 nw417 0 2f
M2981 nw418 nw415 vdd vdd pch w=2u l=180n
M2982 nw418 nw414 vdd vdd pch w=2u l=180n
CT1074 t1074 0 0.1f
M2983 nw418 nw415 t1074 0 nch w=1u l=180n
M2984 t1074 nw414 0 0 nch w=1u l=180n
Cnw418 nw418 0 2f
M2985 nw419 nw417 vdd vdd pch w=2u l=180n
M2986 nw419 nw418 vdd vdd pch w=2u l=180n
CT1075 t1075 0 0.1f
M2987 nw419 nw417 t1075 0 nch w=1u l=180n
M2988 t1075 nw418 0 0 nch w=1u l=180n
Cnw419 nw419 0 2f
CT1076 t1076 0 0.1f
CT1077 t1077 0 0.1f
CT1078 t1078 0 0.1f
M2989 t1076 nw52 vdd vdd pch w=2u l=180n
M2990 t1076 nw349 vdd vdd pch w=2u l=180n
CT1079 t1079 0 0.1f
M2991 t1076 nw52 t1079 0 nch w=1u l=180n
M2992 t1079 nw349 0 0 nch w=1u l=180n
M2993 t1077 nw52 vdd vdd pch w=2u l=180n
M2994 t1077 t1076 vdd vdd pch w=2u l=180n
CT1080 t1080 0 0.1f
M2995 t1077 nw52 t1080 0 nch w=1u l=180n
M2996 t1080 t1076 0 0 nch w=1u l=180n
M2997 t1078 nw349 vdd vdd pch w=2u l=180n
M2998 t1078 t1076 vdd vdd pch w=2u l=180n
CT1081 t1081 0 0.1f
M2999 t1078 nw349 t1081 0 nch w=1u l=180n
M3000 t1081 t1076 0 0 nch w=1u l=180n
M3001 nw420 t1077 vdd vdd pch w=2u l=180n
M3002 nw420 t1078 vdd vdd pch w=2u l=180n
CT1082 t1082 0 0.1f
M3003 nw420 t1077 t1082 0 nch w=1u l=180n
M3004 t1082 t1078 0 0 nch w=1u l=180n
Cnw420 nw420 0 2f
CT1083 t1083 0 0.1f
CT1084 t1084 0 0.1f
CT1085 t1085 0 0.1f
M3005 t1083 nw420 vdd vdd pch w=2u l=180n
M3006 t1083 nw419 vdd vdd pch w=2u l=180n
CT1086 t1086 0 0.1f
M3007 t1083 nw420 t1086 0 nch w=1u l=180n
M3008 t1086 nw419 0 0 nch w=1u l=180n
M3009 t1084 nw420 vdd vdd pch w=2u l=180n
M3010 t1084 t1083 vdd vdd pch w=2u l=180n
CT1087 t1087 0 0.1f
M3011 t1084 nw420 t1087 0 nch w=1u l=180n
M3012 t1087 t1083 0 0 nch w=1u l=180n
M3013 t1085 nw419 vdd vdd pch w=2u l=180n
M3014 t1085 t1083 vdd vdd pch w=2u l=180n
CT1088 t1088 0 0.1f
M3015 t1085 nw419 t1088 0 nch w=1u l=180n
M3016 t1088 t1083 0 0 nch w=1u l=180n
M3017 nw421 t1084 vdd vdd pch w=2u l=180n
M3018 nw421 t1085 vdd vdd pch w=2u l=180n
CT1089 t1089 0 0.1f
M3019 nw421 t1084 t1089 0 nch w=1u l=180n
M3020 t1089 t1085 0 0 nch w=1u l=180n
Cnw421 nw421 0 2f
M3021 nw422 nw52 vdd vdd pch w=2u l=180n
M3022 nw422 nw349 vdd vdd pch w=2u l=180n
CT1090 t1090 0 0.1f
M3023 nw422 nw52 t1090 0 nch w=1u l=180n
M3024 t1090 nw349 0 0 nch w=1u l=180n
Cnw422 nw422 0 2f
M3025 nw423 nw420 vdd vdd pch w=2u l=180n
M3026 nw423 nw419 vdd vdd pch w=2u l=180n
CT1091 t1091 0 0.1f
M3027 nw423 nw420 t1091 0 nch w=1u l=180n
M3028 t1091 nw419 0 0 nch w=1u l=180n
Cnw423 nw423 0 2f
M3029 nw424 nw422 vdd vdd pch w=2u l=180n
M3030 nw424 nw423 vdd vdd pch w=2u l=180n
CT1092 t1092 0 0.1f
M3031 nw424 nw422 t1092 0 nch w=1u l=180n
M3032 t1092 nw423 0 0 nch w=1u l=180n
Cnw424 nw424 0 2f
CT1093 t1093 0 0.1f
CT1094 t1094 0 0.1f
CT1095 t1095 0 0.1f
M3033 t1093 nw53 vdd vdd pch w=2u l=180n
M3034 t1093 nw354 vdd vdd pch w=2u l=180n
CT1096 t1096 0 0.1f
M3035 t1093 nw53 t1096 0 nch w=1u l=180n
M3036 t1096 nw354 0 0 nch w=1u l=180n
M3037 t1094 nw53 vdd vdd pch w=2u l=180n
M3038 t1094 t1093 vdd vdd pch w=2u l=180n
CT1097 t1097 0 0.1f
M3039 t1094 nw53 t1097 0 nch w=1u l=180n
M3040 t1097 t1093 0 0 nch w=1u l=180n
M3041 t1095 nw354 vdd vdd pch w=2u l=180n
M3042 t1095 t1093 vdd vdd pch w=2u l=180n
CT1098 t1098 0 0.1f
M3043 t1095 nw354 t1098 0 nch w=1u l=180n
M3044 t1098 t1093 0 0 nch w=1u l=180n
M3045 nw425 t1094 vdd vdd pch w=2u l=180n
M3046 nw425 t1095 vdd vdd pch w=2u l=180n
CT1099 t1099 0 0.1f
M3047 nw425 t1094 t1099 0 nch w=1u l=180n
M3048 t1099 t1095 0 0 nch w=1u l=180n
Cnw425 nw425 0 2f
CT1100 t1100 0 0.1f
CT1101 t1101 0 0.1f
CT1102 t1102 0 0.1f
M3049 t1100 nw425 vdd vdd pch w=2u l=180n
M3050 t1100 nw424 vdd vdd pch w=2u l=180n
CT1103 t1103 0 0.1f
M3051 t1100 nw425 t1103 0 nch w=1u l=180n
M3052 t1103 nw424 0 0 nch w=1u l=180n
M3053 t1101 nw425 vdd vdd pch w=2u l=180n
M3054 t1101 t1100 vdd vdd pch w=2u l=180n
CT1104 t1104 0 0.1f
M3055 t1101 nw425 t1104 0 nch w=1u l=180n
M3056 t1104 t1100 0 0 nch w=1u l=180n
M3057 t1102 nw424 vdd vdd pch w=2u l=180n
M3058 t1102 t1100 vdd vdd pch w=2u l=180n
CT1105 t1105 0 0.1f
M3059 t1102 nw424 t1105 0 nch w=1u l=180n
M3060 t1105 t1100 0 0 nch w=1u l=180n
M3061 nw426 t1101 vdd vdd pch w=2u l=180n
M3062 nw426 t1102 vdd vdd pch w=2u l=180n
CT1106 t1106 0 0.1f
M3063 nw426 t1101 t1106 0 nch w=1u l=180n
M3064 t1106 t1102 0 0 nch w=1u l=180n
Cnw426 nw426 0 2f
M3065 nw427 nw53 vdd vdd pch w=2u l=180n
M3066 nw427 nw354 vdd vdd pch w=2u l=180n
CT1107 t1107 0 0.1f
M3067 nw427 nw53 t1107 0 nch w=1u l=180n
M3068 t1107 nw354 0 0 nch w=1u l=180n
Cnw427 nw427 0 2f
M3069 nw428 nw425 vdd vdd pch w=2u l=180n
M3070 nw428 nw424 vdd vdd pch w=2u l=180n
CT1108 t1108 0 0.1f
M3071 nw428 nw425 t1108 0 nch w=1u l=180n
M3072 t1108 nw424 0 0 nch w=1u l=180n
Cnw428 nw428 0 2f
M3073 nw429 nw427 vdd vdd pch w=2u l=180n
M3074 nw429 nw428 vdd vdd pch w=2u l=180n
CT1109 t1109 0 0.1f
M3075 nw429 nw427 t1109 0 nch w=1u l=180n
M3076 t1109 nw428 0 0 nch w=1u l=180n
Cnw429 nw429 0 2f
CT1110 t1110 0 0.1f
CT1111 t1111 0 0.1f
CT1112 t1112 0 0.1f
M3077 t1110 nw54 vdd vdd pch w=2u l=180n
M3078 t1110 nw359 vdd vdd pch w=2u l=180n
CT1113 t1113 0 0.1f
M3079 t1110 nw54 t1113 0 nch w=1u l=180n
M3080 t1113 nw359 0 0 nch w=1u l=180n
M3081 t1111 nw54 vdd vdd pch w=2u l=180n
M3082 t1111 t1110 vdd vdd pch w=2u l=180n
CT1114 t1114 0 0.1f
M3083 t1111 nw54 t1114 0 nch w=1u l=180n
M3084 t1114 t1110 0 0 nch w=1u l=180n
M3085 t1112 nw359 vdd vdd pch w=2u l=180n
M3086 t1112 t1110 vdd vdd pch w=2u l=180n
CT1115 t1115 0 0.1f
M3087 t1112 nw359 t1115 0 nch w=1u l=180n
M3088 t1115 t1110 0 0 nch w=1u l=180n
M3089 nw430 t1111 vdd vdd pch w=2u l=180n
M3090 nw430 t1112 vdd vdd pch w=2u l=180n
CT1116 t1116 0 0.1f
M3091 nw430 t1111 t1116 0 nch w=1u l=180n
M3092 t1116 t1112 0 0 nch w=1u l=180n
Cnw430 nw430 0 2f
CT1117 t1117 0 0.1f
CT1118 t1118 0 0.1f
CT1119 t1119 0 0.1f
M3093 t1117 nw430 vdd vdd pch w=2u l=180n
M3094 t1117 nw429 vdd vdd pch w=2u l=180n
CT1120 t1120 0 0.1f
M3095 t1117 nw430 t1120 0 nch w=1u l=180n
M3096 t1120 nw429 0 0 nch w=1u l=180n
M3097 t1118 nw430 vdd vdd pch w=2u l=180n
M3098 t1118 t1117 vdd vdd pch w=2u l=180n
CT1121 t1121 0 0.1f
M3099 t1118 nw430 t1121 0 nch w=1u l=180n
M3100 t1121 t1117 0 0 nch w=1u l=180n
M3101 t1119 nw429 vdd vdd pch w=2u l=180n
M3102 t1119 t1117 vdd vdd pch w=2u l=180n
CT1122 t1122 0 0.1f
M3103 t1119 nw429 t1122 0 nch w=1u l=180n
M3104 t1122 t1117 0 0 nch w=1u l=180n
M3105 nw431 t1118 vdd vdd pch w=2u l=180n
M3106 nw431 t1119 vdd vdd pch w=2u l=180n
CT1123 t1123 0 0.1f
M3107 nw431 t1118 t1123 0 nch w=1u l=180n
M3108 t1123 t1119 0 0 nch w=1u l=180n
Cnw431 nw431 0 2f
M3109 nw432 nw54 vdd vdd pch w=2u l=180n
M3110 nw432 nw359 vdd vdd pch w=2u l=180n
CT1124 t1124 0 0.1f
M3111 nw432 nw54 t1124 0 nch w=1u l=180n
M3112 t1124 nw359 0 0 nch w=1u l=180n
Cnw432 nw432 0 2f
M3113 nw433 nw430 vdd vdd pch w=2u l=180n
M3114 nw433 nw429 vdd vdd pch w=2u l=180n
CT1125 t1125 0 0.1f
M3115 nw433 nw430 t1125 0 nch w=1u l=180n
M3116 t1125 nw429 0 0 nch w=1u l=180n
Cnw433 nw433 0 2f
M3117 nw434 nw432 vdd vdd pch w=2u l=180n
M3118 nw434 nw433 vdd vdd pch w=2u l=180n
CT1126 t1126 0 0.1f
M3119 nw434 nw432 t1126 0 nch w=1u l=180n
M3120 t1126 nw433 0 0 nch w=1u l=180n
Cnw434 nw434 0 2f
CT1127 t1127 0 0.1f
CT1128 t1128 0 0.1f
CT1129 t1129 0 0.1f
M3121 t1127 nw55 vdd vdd pch w=2u l=180n
M3122 t1127 nw364 vdd vdd pch w=2u l=180n
CT1130 t1130 0 0.1f
M3123 t1127 nw55 t1130 0 nch w=1u l=180n
M3124 t1130 nw364 0 0 nch w=1u l=180n
M3125 t1128 nw55 vdd vdd pch w=2u l=180n
M3126 t1128 t1127 vdd vdd pch w=2u l=180n
CT1131 t1131 0 0.1f
M3127 t1128 nw55 t1131 0 nch w=1u l=180n
M3128 t1131 t1127 0 0 nch w=1u l=180n
M3129 t1129 nw364 vdd vdd pch w=2u l=180n
M3130 t1129 t1127 vdd vdd pch w=2u l=180n
CT1132 t1132 0 0.1f
M3131 t1129 nw364 t1132 0 nch w=1u l=180n
M3132 t1132 t1127 0 0 nch w=1u l=180n
M3133 nw435 t1128 vdd vdd pch w=2u l=180n
M3134 nw435 t1129 vdd vdd pch w=2u l=180n
CT1133 t1133 0 0.1f
M3135 nw435 t1128 t1133 0 nch w=1u l=180n
M3136 t1133 t1129 0 0 nch w=1u l=180n
Cnw435 nw435 0 2f
CT1134 t1134 0 0.1f
CT1135 t1135 0 0.1f
CT1136 t1136 0 0.1f
M3137 t1134 nw435 vdd vdd pch w=2u l=180n
M3138 t1134 nw434 vdd vdd pch w=2u l=180n
CT1137 t1137 0 0.1f
M3139 t1134 nw435 t1137 0 nch w=1u l=180n
M3140 t1137 nw434 0 0 nch w=1u l=180n
M3141 t1135 nw435 vdd vdd pch w=2u l=180n
M3142 t1135 t1134 vdd vdd pch w=2u l=180n
CT1138 t1138 0 0.1f
M3143 t1135 nw435 t1138 0 nch w=1u l=180n
M3144 t1138 t1134 0 0 nch w=1u l=180n
M3145 t1136 nw434 vdd vdd pch w=2u l=180n
M3146 t1136 t1134 vdd vdd pch w=2u l=180n
CT1139 t1139 0 0.1f
M3147 t1136 nw434 t1139 0 nch w=1u l=180n
M3148 t1139 t1134 0 0 nch w=1u l=180n
M3149 nw436 t1135 vdd vdd pch w=2u l=180n
M3150 nw436 t1136 vdd vdd pch w=2u l=180n
CT1140 t1140 0 0.1f
M3151 nw436 t1135 t1140 0 nch w=1u l=180n
M3152 t1140 t1136 0 0 nch w=1u l=180n
Cnw436 nw436 0 2f
M3153 nw437 nw55 vdd vdd pch w=2u l=180n
M3154 nw437 nw364 vdd vdd pch w=2u l=180n
CT1141 t1141 0 0.1f
M3155 nw437 nw55 t1141 0 nch w=1u l=180n
M3156 t1141 nw364 0 0 nch w=1u l=180n
Cnw437 nw437 0 2f
M3157 nw438 nw435 vdd vdd pch w=2u l=180n
M3158 nw438 nw434 vdd vdd pch w=2u l=180n
CT1142 t1142 0 0.1f
M3159 nw438 nw435 t1142 0 nch w=1u l=180n
M3160 t1142 nw434 0 0 nch w=1u l=180n
Cnw438 nw438 0 2f
M3161 nw439 nw437 vdd vdd pch w=2u l=180n
M3162 nw439 nw438 vdd vdd pch w=2u l=180n
CT1143 t1143 0 0.1f
M3163 nw439 nw437 t1143 0 nch w=1u l=180n
M3164 t1143 nw438 0 0 nch w=1u l=180n
Cnw439 nw439 0 2f
CT1144 t1144 0 0.1f
CT1145 t1145 0 0.1f
CT1146 t1146 0 0.1f
M3165 t1144 nw56 vdd vdd pch w=2u l=180n
M3166 t1144 nw369 vdd vdd pch w=2u l=180n
CT1147 t1147 0 0.1f
M3167 t1144 nw56 t1147 0 nch w=1u l=180n
M3168 t1147 nw369 0 0 nch w=1u l=180n
M3169 t1145 nw56 vdd vdd pch w=2u l=180n
M3170 t1145 t1144 vdd vdd pch w=2u l=180n
CT1148 t1148 0 0.1f
M3171 t1145 nw56 t1148 0 nch w=1u l=180n
M3172 t1148 t1144 0 0 nch w=1u l=180n
M3173 t1146 nw369 vdd vdd pch w=2u l=180n
M3174 t1146 t1144 vdd vdd pch w=2u l=180n
CT1149 t1149 0 0.1f
M3175 t1146 nw369 t1149 0 nch w=1u l=180n
M3176 t1149 t1144 0 0 nch w=1u l=180n
M3177 nw440 t1145 vdd vdd pch w=2u l=180n
M3178 nw440 t1146 vdd vdd pch w=2u l=180n
CT1150 t1150 0 0.1f
M3179 nw440 t1145 t1150 0 nch w=1u l=180n
M3180 t1150 t1146 0 0 nch w=1u l=180n
Cnw440 nw440 0 2f
CT1151 t1151 0 0.1f
CT1152 t1152 0 0.1f
CT1153 t1153 0 0.1f
M3181 t1151 nw440 vdd vdd pch w=2u l=180n
M3182 t1151 nw439 vdd vdd pch w=2u l=180n
CT1154 t1154 0 0.1f
M3183 t1151 nw440 t1154 0 nch w=1u l=180n
M3184 t1154 nw439 0 0 nch w=1u l=180n
M3185 t1152 nw440 vdd vdd pch w=2u l=180n
M3186 t1152 t1151 vdd vdd pch w=2u l=180n
CT1155 t1155 0 0.1f
M3187 t1152 nw440 t1155 0 nch w=1u l=180n
M3188 t1155 t1151 0 0 nch w=1u l=180n
M3189 t1153 nw439 vdd vdd pch w=2u l=180n
M3190 t1153 t1151 vdd vdd pch w=2u l=180n
CT1156 t1156 0 0.1f
M3191 t1153 nw439 t1156 0 nch w=1u l=180n
M3192 t1156 t1151 0 0 nch w=1u l=180n
M3193 nw441 t1152 vdd vdd pch w=2u l=180n
M3194 nw441 t1153 vdd vdd pch w=2u l=180n
CT1157 t1157 0 0.1f
M3195 nw441 t1152 t1157 0 nch w=1u l=180n
M3196 t1157 t1153 0 0 nch w=1u l=180n
Cnw441 nw441 0 2f
M3197 nw442 nw56 vdd vdd pch w=2u l=180n
M3198 nw442 nw369 vdd vdd pch w=2u l=180n
CT1158 t1158 0 0.1f
M3199 nw442 nw56 t1158 0 nch w=1u l=180n
M3200 t1158 nw369 0 0 nch w=1u l=180n
Cnw442 nw442 0 2f
M3201 nw443 nw440 vdd vdd pch w=2u l=180n
M3202 nw443 nw439 vdd vdd pch w=2u l=180n
CT1159 t1159 0 0.1f
M3203 nw443 nw440 t1159 0 nch w=1u l=180n
M3204 t1159 nw439 0 0 nch w=1u l=180n
Cnw443 nw443 0 2f
M3205 nw444 nw442 vdd vdd pch w=2u l=180n
M3206 nw444 nw443 vdd vdd pch w=2u l=180n
CT1160 t1160 0 0.1f
M3207 nw444 nw442 t1160 0 nch w=1u l=180n
M3208 t1160 nw443 0 0 nch w=1u l=180n
Cnw444 nw444 0 2f
CT1161 t1161 0 0.1f
CT1162 t1162 0 0.1f
CT1163 t1163 0 0.1f
M3209 t1161 nw57 vdd vdd pch w=2u l=180n
M3210 t1161 nw374 vdd vdd pch w=2u l=180n
CT1164 t1164 0 0.1f
M3211 t1161 nw57 t1164 0 nch w=1u l=180n
M3212 t1164 nw374 0 0 nch w=1u l=180n
M3213 t1162 nw57 vdd vdd pch w=2u l=180n
M3214 t1162 t1161 vdd vdd pch w=2u l=180n
CT1165 t1165 0 0.1f
M3215 t1162 nw57 t1165 0 nch w=1u l=180n
M3216 t1165 t1161 0 0 nch w=1u l=180n
M3217 t1163 nw374 vdd vdd pch w=2u l=180n
M3218 t1163 t1161 vdd vdd pch w=2u l=180n
CT1166 t1166 0 0.1f
M3219 t1163 nw374 t1166 0 nch w=1u l=180n
M3220 t1166 t1161 0 0 nch w=1u l=180n
M3221 nw445 t1162 vdd vdd pch w=2u l=180n
M3222 nw445 t1163 vdd vdd pch w=2u l=180n
CT1167 t1167 0 0.1f
M3223 nw445 t1162 t1167 0 nch w=1u l=180n
M3224 t1167 t1163 0 0 nch w=1u l=180n
Cnw445 nw445 0 2f
CT1168 t1168 0 0.1f
CT1169 t1169 0 0.1f
CT1170 t1170 0 0.1f
M3225 t1168 nw445 vdd vdd pch w=2u l=180n
M3226 t1168 nw444 vdd vdd pch w=2u l=180n
CT1171 t1171 0 0.1f
M3227 t1168 nw445 t1171 0 nch w=1u l=180n
M3228 t1171 nw444 0 0 nch w=1u l=180n
M3229 t1169 nw445 vdd vdd pch w=2u l=180n
M3230 t1169 t1168 vdd vdd pch w=2u l=180n
CT1172 t1172 0 0.1f
M3231 t1169 nw445 t1172 0 nch w=1u l=180n
M3232 t1172 t1168 0 0 nch w=1u l=180n
M3233 t1170 nw444 vdd vdd pch w=2u l=180n
M3234 t1170 t1168 vdd vdd pch w=2u l=180n
CT1173 t1173 0 0.1f
M3235 t1170 nw444 t1173 0 nch w=1u l=180n
M3236 t1173 t1168 0 0 nch w=1u l=180n
M3237 nw446 t1169 vdd vdd pch w=2u l=180n
M3238 nw446 t1170 vdd vdd pch w=2u l=180n
CT1174 t1174 0 0.1f
M3239 nw446 t1169 t1174 0 nch w=1u l=180n
M3240 t1174 t1170 0 0 nch w=1u l=180n
Cnw446 nw446 0 2f
M3241 nw447 nw57 vdd vdd pch w=2u l=180n
M3242 nw447 nw374 vdd vdd pch w=2u l=180n
CT1175 t1175 0 0.1f
M3243 nw447 nw57 t1175 0 nch w=1u l=180n
M3244 t1175 nw374 0 0 nch w=1u l=180n
Cnw447 nw447 0 2f
M3245 nw448 nw445 vdd vdd pch w=2u l=180n
M3246 nw448 nw444 vdd vdd pch w=2u l=180n
CT1176 t1176 0 0.1f
M3247 nw448 nw445 t1176 0 nch w=1u l=180n
M3248 t1176 nw444 0 0 nch w=1u l=180n
Cnw448 nw448 0 2f
M3249 nw449 nw447 vdd vdd pch w=2u l=180n
M3250 nw449 nw448 vdd vdd pch w=2u l=180n
CT1177 t1177 0 0.1f
M3251 nw449 nw447 t1177 0 nch w=1u l=180n
M3252 t1177 nw448 0 0 nch w=1u l=180n
Cnw449 nw449 0 2f
CT1178 t1178 0 0.1f
CT1179 t1179 0 0.1f
CT1180 t1180 0 0.1f
M3253 t1178 nw58 vdd vdd pch w=2u l=180n
M3254 t1178 nw379 vdd vdd pch w=2u l=180n
CT1181 t1181 0 0.1f
M3255 t1178 nw58 t1181 0 nch w=1u l=180n
M3256 t1181 nw379 0 0 nch w=1u l=180n
M3257 t1179 nw58 vdd vdd pch w=2u l=180n
M3258 t1179 t1178 vdd vdd pch w=2u l=180n
CT1182 t1182 0 0.1f
M3259 t1179 nw58 t1182 0 nch w=1u l=180n
M3260 t1182 t1178 0 0 nch w=1u l=180n
M3261 t1180 nw379 vdd vdd pch w=2u l=180n
M3262 t1180 t1178 vdd vdd pch w=2u l=180n
CT1183 t1183 0 0.1f
M3263 t1180 nw379 t1183 0 nch w=1u l=180n
M3264 t1183 t1178 0 0 nch w=1u l=180n
M3265 nw450 t1179 vdd vdd pch w=2u l=180n
M3266 nw450 t1180 vdd vdd pch w=2u l=180n
CT1184 t1184 0 0.1f
M3267 nw450 t1179 t1184 0 nch w=1u l=180n
M3268 t1184 t1180 0 0 nch w=1u l=180n
Cnw450 nw450 0 2f
CT1185 t1185 0 0.1f
CT1186 t1186 0 0.1f
CT1187 t1187 0 0.1f
M3269 t1185 nw450 vdd vdd pch w=2u l=180n
M3270 t1185 nw449 vdd vdd pch w=2u l=180n
CT1188 t1188 0 0.1f
M3271 t1185 nw450 t1188 0 nch w=1u l=180n
M3272 t1188 nw449 0 0 nch w=1u l=180n
M3273 t1186 nw450 vdd vdd pch w=2u l=180n
M3274 t1186 t1185 vdd vdd pch w=2u l=180n
CT1189 t1189 0 0.1f
M3275 t1186 nw450 t1189 0 nch w=1u l=180n
M3276 t1189 t1185 0 0 nch w=1u l=180n
M3277 t1187 nw449 vdd vdd pch w=2u l=180n
M3278 t1187 t1185 vdd vdd pch w=2u l=180n
CT1190 t1190 0 0.1f
M3279 t1187 nw449 t1190 0 nch w=1u l=180n
M3280 t1190 t1185 0 0 nch w=1u l=180n
M3281 nw451 t1186 vdd vdd pch w=2u l=180n
M3282 nw451 t1187 vdd vdd pch w=2u l=180n
CT1191 t1191 0 0.1f
M3283 nw451 t1186 t1191 0 nch w=1u l=180n
M3284 t1191 t1187 0 0 nch w=1u l=180n
Cnw451 nw451 0 2f
M3285 nw452 nw58 vdd vdd pch w=2u l=180n
M3286 nw452 nw379 vdd vdd pch w=2u l=180n
CT1192 t1192 0 0.1f
M3287 nw452 nw58 t1192 0 nch w=1u l=180n
M3288 t1192 nw379 0 0 nch w=1u l=180n
Cnw452 nw452 0 2f
M3289 nw453 nw450 vdd vdd pch w=2u l=180n
M3290 nw453 nw449 vdd vdd pch w=2u l=180n
CT1193 t1193 0 0.1f
M3291 nw453 nw450 t1193 0 nch w=1u l=180n
M3292 t1193 nw449 0 0 nch w=1u l=180n
Cnw453 nw453 0 2f
M3293 nw454 nw452 vdd vdd pch w=2u l=180n
M3294 nw454 nw453 vdd vdd pch w=2u l=180n
CT1194 t1194 0 0.1f
M3295 nw454 nw452 t1194 0 nch w=1u l=180n
M3296 t1194 nw453 0 0 nch w=1u l=180n
Cnw454 nw454 0 2f
CT1195 t1195 0 0.1f
CT1196 t1196 0 0.1f
CT1197 t1197 0 0.1f
M3297 t1195 nw59 vdd vdd pch w=2u l=180n
M3298 t1195 nw384 vdd vdd pch w=2u l=180n
CT1198 t1198 0 0.1f
M3299 t1195 nw59 t1198 0 nch w=1u l=180n
M3300 t1198 nw384 0 0 nch w=1u l=180n
M3301 t1196 nw59 vdd vdd pch w=2u l=180n
M3302 t1196 t1195 vdd vdd pch w=2u l=180n
CT1199 t1199 0 0.1f
M3303 t1196 nw59 t1199 0 nch w=1u l=180n
M3304 t1199 t1195 0 0 nch w=1u l=180n
M3305 t1197 nw384 vdd vdd pch w=2u l=180n
M3306 t1197 t1195 vdd vdd pch w=2u l=180n
CT1200 t1200 0 0.1f
M3307 t1197 nw384 t1200 0 nch w=1u l=180n
M3308 t1200 t1195 0 0 nch w=1u l=180n
M3309 nw455 t1196 vdd vdd pch w=2u l=180n
M3310 nw455 t1197 vdd vdd pch w=2u l=180n
CT1201 t1201 0 0.1f
M3311 nw455 t1196 t1201 0 nch w=1u l=180n
M3312 t1201 t1197 0 0 nch w=1u l=180n
Cnw455 nw455 0 2f
CT1202 t1202 0 0.1f
CT1203 t1203 0 0.1f
CT1204 t1204 0 0.1f
M3313 t1202 nw455 vdd vdd pch w=2u l=180n
M3314 t1202 nw454 vdd vdd pch w=2u l=180n
CT1205 t1205 0 0.1f
M3315 t1202 nw455 t1205 0 nch w=1u l=180n
M3316 t1205 nw454 0 0 nch w=1u l=180n
M3317 t1203 nw455 vdd vdd pch w=2u l=180n
M3318 t1203 t1202 vdd vdd pch w=2u l=180n
CT1206 t1206 0 0.1f
M3319 t1203 nw455 t1206 0 nch w=1u l=180n
M3320 t1206 t1202 0 0 nch w=1u l=180n
M3321 t1204 nw454 vdd vdd pch w=2u l=180n
M3322 t1204 t1202 vdd vdd pch w=2u l=180n
CT1207 t1207 0 0.1f
M3323 t1204 nw454 t1207 0 nch w=1u l=180n
M3324 t1207 t1202 0 0 nch w=1u l=180n
M3325 nw456 t1203 vdd vdd pch w=2u l=180n
M3326 nw456 t1204 vdd vdd pch w=2u l=180n
CT1208 t1208 0 0.1f
M3327 nw456 t1203 t1208 0 nch w=1u l=180n
M3328 t1208 t1204 0 0 nch w=1u l=180n
Cnw456 nw456 0 2f
M3329 nw457 nw59 vdd vdd pch w=2u l=180n
M3330 nw457 nw384 vdd vdd pch w=2u l=180n
CT1209 t1209 0 0.1f
M3331 nw457 nw59 t1209 0 nch w=1u l=180n
M3332 t1209 nw384 0 0 nch w=1u l=180n
Cnw457 nw457 0 2f
M3333 nw458 nw455 vdd vdd pch w=2u l=180n
M3334 nw458 nw454 vdd vdd pch w=2u l=180n
CT1210 t1210 0 0.1f
M3335 nw458 nw455 t1210 0 nch w=1u l=180n
M3336 t1210 nw454 0 0 nch w=1u l=180n
Cnw458 nw458 0 2f
M3337 nw459 nw457 vdd vdd pch w=2u l=180n
M3338 nw459 nw458 vdd vdd pch w=2u l=180n
CT1211 t1211 0 0.1f
M3339 nw459 nw457 t1211 0 nch w=1u l=180n
M3340 t1211 nw458 0 0 nch w=1u l=180n
Cnw459 nw459 0 2f
CT1212 t1212 0 0.1f
CT1213 t1213 0 0.1f
CT1214 t1214 0 0.1f
M3341 t1212 nw60 vdd vdd pch w=2u l=180n
M3342 t1212 nw389 vdd vdd pch w=2u l=180n
CT1215 t1215 0 0.1f
M3343 t1212 nw60 t1215 0 nch w=1u l=180n
M3344 t1215 nw389 0 0 nch w=1u l=180n
M3345 t1213 nw60 vdd vdd pch w=2u l=180n
M3346 t1213 t1212 vdd vdd pch w=2u l=180n
CT1216 t1216 0 0.1f
M3347 t1213 nw60 t1216 0 nch w=1u l=180n
M3348 t1216 t1212 0 0 nch w=1u l=180n
M3349 t1214 nw389 vdd vdd pch w=2u l=180n
M3350 t1214 t1212 vdd vdd pch w=2u l=180n
CT1217 t1217 0 0.1f
M3351 t1214 nw389 t1217 0 nch w=1u l=180n
M3352 t1217 t1212 0 0 nch w=1u l=180n
M3353 nw460 t1213 vdd vdd pch w=2u l=180n
M3354 nw460 t1214 vdd vdd pch w=2u l=180n
CT1218 t1218 0 0.1f
M3355 nw460 t1213 t1218 0 nch w=1u l=180n
M3356 t1218 t1214 0 0 nch w=1u l=180n
Cnw460 nw460 0 2f
CT1219 t1219 0 0.1f
CT1220 t1220 0 0.1f
CT1221 t1221 0 0.1f
M3357 t1219 nw460 vdd vdd pch w=2u l=180n
M3358 t1219 nw459 vdd vdd pch w=2u l=180n
CT1222 t1222 0 0.1f
M3359 t1219 nw460 t1222 0 nch w=1u l=180n
M3360 t1222 nw459 0 0 nch w=1u l=180n
M3361 t1220 nw460 vdd vdd pch w=2u l=180n
M3362 t1220 t1219 vdd vdd pch w=2u l=180n
CT1223 t1223 0 0.1f
M3363 t1220 nw460 t1223 0 nch w=1u l=180n
M3364 t1223 t1219 0 0 nch w=1u l=180n
M3365 t1221 nw459 vdd vdd pch w=2u l=180n
M3366 t1221 t1219 vdd vdd pch w=2u l=180n
CT1224 t1224 0 0.1f
M3367 t1221 nw459 t1224 0 nch w=1u l=180n
M3368 t1224 t1219 0 0 nch w=1u l=180n
M3369 nw461 t1220 vdd vdd pch w=2u l=180n
M3370 nw461 t1221 vdd vdd pch w=2u l=180n
CT1225 t1225 0 0.1f
M3371 nw461 t1220 t1225 0 nch w=1u l=180n
M3372 t1225 t1221 0 0 nch w=1u l=180n
Cnw461 nw461 0 2f
M3373 nw462 nw60 vdd vdd pch w=2u l=180n
M3374 nw462 nw389 vdd vdd pch w=2u l=180n
CT1226 t1226 0 0.1f
M3375 nw462 nw60 t1226 0 nch w=1u l=180n
M3376 t1226 nw389 0 0 nch w=1u l=180n
Cnw462 nw462 0 2f
M3377 nw463 nw460 vdd vdd pch w=2u l=180n
M3378 nw463 nw459 vdd vdd pch w=2u l=180n
CT1227 t1227 0 0.1f
M3379 nw463 nw460 t1227 0 nch w=1u l=180n
M3380 t1227 nw459 0 0 nch w=1u l=180n
Cnw463 nw463 0 2f
M3381 nw464 nw462 vdd vdd pch w=2u l=180n
M3382 nw464 nw463 vdd vdd pch w=2u l=180n
CT1228 t1228 0 0.1f
M3383 nw464 nw462 t1228 0 nch w=1u l=180n
M3384 t1228 nw463 0 0 nch w=1u l=180n
Cnw464 nw464 0 2f
CT1229 t1229 0 0.1f
CT1230 t1230 0 0.1f
CT1231 t1231 0 0.1f
M3385 t1229 nw61 vdd vdd pch w=2u l=180n
M3386 t1229 nw394 vdd vdd pch w=2u l=180n
CT1232 t1232 0 0.1f
M3387 t1229 nw61 t1232 0 nch w=1u l=180n
M3388 t1232 nw394 0 0 nch w=1u l=180n
M3389 t1230 nw61 vdd vdd pch w=2u l=180n
M3390 t1230 t1229 vdd vdd pch w=2u l=180n
CT1233 t1233 0 0.1f
M3391 t1230 nw61 t1233 0 nch w=1u l=180n
M3392 t1233 t1229 0 0 nch w=1u l=180n
M3393 t1231 nw394 vdd vdd pch w=2u l=180n
M3394 t1231 t1229 vdd vdd pch w=2u l=180n
CT1234 t1234 0 0.1f
M3395 t1231 nw394 t1234 0 nch w=1u l=180n
M3396 t1234 t1229 0 0 nch w=1u l=180n
M3397 nw465 t1230 vdd vdd pch w=2u l=180n
M3398 nw465 t1231 vdd vdd pch w=2u l=180n
CT1235 t1235 0 0.1f
M3399 nw465 t1230 t1235 0 nch w=1u l=180n
M3400 t1235 t1231 0 0 nch w=1u l=180n
Cnw465 nw465 0 2f
CT1236 t1236 0 0.1f
CT1237 t1237 0 0.1f
CT1238 t1238 0 0.1f
M3401 t1236 nw465 vdd vdd pch w=2u l=180n
M3402 t1236 nw464 vdd vdd pch w=2u l=180n
CT1239 t1239 0 0.1f
M3403 t1236 nw465 t1239 0 nch w=1u l=180n
M3404 t1239 nw464 0 0 nch w=1u l=180n
M3405 t1237 nw465 vdd vdd pch w=2u l=180n
M3406 t1237 t1236 vdd vdd pch w=2u l=180n
CT1240 t1240 0 0.1f
M3407 t1237 nw465 t1240 0 nch w=1u l=180n
M3408 t1240 t1236 0 0 nch w=1u l=180n
M3409 t1238 nw464 vdd vdd pch w=2u l=180n
M3410 t1238 t1236 vdd vdd pch w=2u l=180n
CT1241 t1241 0 0.1f
M3411 t1238 nw464 t1241 0 nch w=1u l=180n
M3412 t1241 t1236 0 0 nch w=1u l=180n
M3413 nw466 t1237 vdd vdd pch w=2u l=180n
M3414 nw466 t1238 vdd vdd pch w=2u l=180n
CT1242 t1242 0 0.1f
M3415 nw466 t1237 t1242 0 nch w=1u l=180n
M3416 t1242 t1238 0 0 nch w=1u l=180n
Cnw466 nw466 0 2f
M3417 nw467 nw61 vdd vdd pch w=2u l=180n
M3418 nw467 nw394 vdd vdd pch w=2u l=180n
CT1243 t1243 0 0.1f
M3419 nw467 nw61 t1243 0 nch w=1u l=180n
M3420 t1243 nw394 0 0 nch w=1u l=180n
Cnw467 nw467 0 2f
M3421 nw468 nw465 vdd vdd pch w=2u l=180n
M3422 nw468 nw464 vdd vdd pch w=2u l=180n
CT1244 t1244 0 0.1f
M3423 nw468 nw465 t1244 0 nch w=1u l=180n
M3424 t1244 nw464 0 0 nch w=1u l=180n
Cnw468 nw468 0 2f
M3425 nw469 nw467 vdd vdd pch w=2u l=180n
M3426 nw469 nw468 vdd vdd pch w=2u l=180n
CT1245 t1245 0 0.1f
M3427 nw469 nw467 t1245 0 nch w=1u l=180n
M3428 t1245 nw468 0 0 nch w=1u l=180n
Cnw469 nw469 0 2f
CT1246 t1246 0 0.1f
CT1247 t1247 0 0.1f
CT1248 t1248 0 0.1f
M3429 t1246 nw62 vdd vdd pch w=2u l=180n
M3430 t1246 nw399 vdd vdd pch w=2u l=180n
CT1249 t1249 0 0.1f
M3431 t1246 nw62 t1249 0 nch w=1u l=180n
M3432 t1249 nw399 0 0 nch w=1u l=180n
M3433 t1247 nw62 vdd vdd pch w=2u l=180n
M3434 t1247 t1246 vdd vdd pch w=2u l=180n
CT1250 t1250 0 0.1f
M3435 t1247 nw62 t1250 0 nch w=1u l=180n
M3436 t1250 t1246 0 0 nch w=1u l=180n
M3437 t1248 nw399 vdd vdd pch w=2u l=180n
M3438 t1248 t1246 vdd vdd pch w=2u l=180n
CT1251 t1251 0 0.1f
M3439 t1248 nw399 t1251 0 nch w=1u l=180n
M3440 t1251 t1246 0 0 nch w=1u l=180n
M3441 nw470 t1247 vdd vdd pch w=2u l=180n
M3442 nw470 t1248 vdd vdd pch w=2u l=180n
CT1252 t1252 0 0.1f
M3443 nw470 t1247 t1252 0 nch w=1u l=180n
M3444 t1252 t1248 0 0 nch w=1u l=180n
Cnw470 nw470 0 2f
CT1253 t1253 0 0.1f
CT1254 t1254 0 0.1f
CT1255 t1255 0 0.1f
M3445 t1253 nw470 vdd vdd pch w=2u l=180n
M3446 t1253 nw469 vdd vdd pch w=2u l=180n
CT1256 t1256 0 0.1f
M3447 t1253 nw470 t1256 0 nch w=1u l=180n
M3448 t1256 nw469 0 0 nch w=1u l=180n
M3449 t1254 nw470 vdd vdd pch w=2u l=180n
M3450 t1254 t1253 vdd vdd pch w=2u l=180n
CT1257 t1257 0 0.1f
M3451 t1254 nw470 t1257 0 nch w=1u l=180n
M3452 t1257 t1253 0 0 nch w=1u l=180n
M3453 t1255 nw469 vdd vdd pch w=2u l=180n
M3454 t1255 t1253 vdd vdd pch w=2u l=180n
CT1258 t1258 0 0.1f
M3455 t1255 nw469 t1258 0 nch w=1u l=180n
M3456 t1258 t1253 0 0 nch w=1u l=180n
M3457 nw471 t1254 vdd vdd pch w=2u l=180n
M3458 nw471 t1255 vdd vdd pch w=2u l=180n
CT1259 t1259 0 0.1f
M3459 nw471 t1254 t1259 0 nch w=1u l=180n
M3460 t1259 t1255 0 0 nch w=1u l=180n
Cnw471 nw471 0 2f
M3461 nw472 nw62 vdd vdd pch w=2u l=180n
M3462 nw472 nw399 vdd vdd pch w=2u l=180n
CT1260 t1260 0 0.1f
M3463 nw472 nw62 t1260 0 nch w=1u l=180n
M3464 t1260 nw399 0 0 nch w=1u l=180n
Cnw472 nw472 0 2f
M3465 nw473 nw470 vdd vdd pch w=2u l=180n
M3466 nw473 nw469 vdd vdd pch w=2u l=180n
CT1261 t1261 0 0.1f
M3467 nw473 nw470 t1261 0 nch w=1u l=180n
M3468 t1261 nw469 0 0 nch w=1u l=180n
Cnw473 nw473 0 2f
M3469 nw474 nw472 vdd vdd pch w=2u l=180n
M3470 nw474 nw473 vdd vdd pch w=2u l=180n
CT1262 t1262 0 0.1f
M3471 nw474 nw472 t1262 0 nch w=1u l=180n
M3472 t1262 nw473 0 0 nch w=1u l=180n
Cnw474 nw474 0 2f
CT1263 t1263 0 0.1f
CT1264 t1264 0 0.1f
CT1265 t1265 0 0.1f
M3473 t1263 nw63 vdd vdd pch w=2u l=180n
M3474 t1263 nw404 vdd vdd pch w=2u l=180n
CT1266 t1266 0 0.1f
M3475 t1263 nw63 t1266 0 nch w=1u l=180n
M3476 t1266 nw404 0 0 nch w=1u l=180n
M3477 t1264 nw63 vdd vdd pch w=2u l=180n
M3478 t1264 t1263 vdd vdd pch w=2u l=180n
CT1267 t1267 0 0.1f
M3479 t1264 nw63 t1267 0 nch w=1u l=180n
M3480 t1267 t1263 0 0 nch w=1u l=180n
M3481 t1265 nw404 vdd vdd pch w=2u l=180n
M3482 t1265 t1263 vdd vdd pch w=2u l=180n
CT1268 t1268 0 0.1f
M3483 t1265 nw404 t1268 0 nch w=1u l=180n
M3484 t1268 t1263 0 0 nch w=1u l=180n
M3485 nw475 t1264 vdd vdd pch w=2u l=180n
M3486 nw475 t1265 vdd vdd pch w=2u l=180n
CT1269 t1269 0 0.1f
M3487 nw475 t1264 t1269 0 nch w=1u l=180n
M3488 t1269 t1265 0 0 nch w=1u l=180n
Cnw475 nw475 0 2f
CT1270 t1270 0 0.1f
CT1271 t1271 0 0.1f
CT1272 t1272 0 0.1f
M3489 t1270 nw475 vdd vdd pch w=2u l=180n
M3490 t1270 nw474 vdd vdd pch w=2u l=180n
CT1273 t1273 0 0.1f
M3491 t1270 nw475 t1273 0 nch w=1u l=180n
M3492 t1273 nw474 0 0 nch w=1u l=180n
M3493 t1271 nw475 vdd vdd pch w=2u l=180n
M3494 t1271 t1270 vdd vdd pch w=2u l=180n
CT1274 t1274 0 0.1f
M3495 t1271 nw475 t1274 0 nch w=1u l=180n
M3496 t1274 t1270 0 0 nch w=1u l=180n
M3497 t1272 nw474 vdd vdd pch w=2u l=180n
M3498 t1272 t1270 vdd vdd pch w=2u l=180n
CT1275 t1275 0 0.1f
M3499 t1272 nw474 t1275 0 nch w=1u l=180n
M3500 t1275 t1270 0 0 nch w=1u l=180n
M3501 nw476 t1271 vdd vdd pch w=2u l=180n
M3502 nw476 t1272 vdd vdd pch w=2u l=180n
CT1276 t1276 0 0.1f
M3503 nw476 t1271 t1276 0 nch w=1u l=180n
M3504 t1276 t1272 0 0 nch w=1u l=180n
Cnw476 nw476 0 2f
M3505 nw477 nw63 vdd vdd pch w=2u l=180n
M3506 nw477 nw404 vdd vdd pch w=2u l=180n
CT1277 t1277 0 0.1f
M3507 nw477 nw63 t1277 0 nch w=1u l=180n
M3508 t1277 nw404 0 0 nch w=1u l=180n
Cnw477 nw477 0 2f
M3509 nw478 nw475 vdd vdd pch w=2u l=180n
M3510 nw478 nw474 vdd vdd pch w=2u l=180n
CT1278 t1278 0 0.1f
M3511 nw478 nw475 t1278 0 nch w=1u l=180n
M3512 t1278 nw474 0 0 nch w=1u l=180n
Cnw478 nw478 0 2f
M3513 nw479 nw477 vdd vdd pch w=2u l=180n
M3514 nw479 nw478 vdd vdd pch w=2u l=180n
CT1279 t1279 0 0.1f
M3515 nw479 nw477 t1279 0 nch w=1u l=180n
M3516 t1279 nw478 0 0 nch w=1u l=180n
Cnw479 nw479 0 2f
CT1280 t1280 0 0.1f
CT1281 t1281 0 0.1f
CT1282 t1282 0 0.1f
M3517 t1280 nw64 vdd vdd pch w=2u l=180n
M3518 t1280 nw407 vdd vdd pch w=2u l=180n
CT1283 t1283 0 0.1f
M3519 t1280 nw64 t1283 0 nch w=1u l=180n
M3520 t1283 nw407 0 0 nch w=1u l=180n
M3521 t1281 nw64 vdd vdd pch w=2u l=180n
M3522 t1281 t1280 vdd vdd pch w=2u l=180n
CT1284 t1284 0 0.1f
M3523 t1281 nw64 t1284 0 nch w=1u l=180n
M3524 t1284 t1280 0 0 nch w=1u l=180n
M3525 t1282 nw407 vdd vdd pch w=2u l=180n
M3526 t1282 t1280 vdd vdd pch w=2u l=180n
CT1285 t1285 0 0.1f
M3527 t1282 nw407 t1285 0 nch w=1u l=180n
M3528 t1285 t1280 0 0 nch w=1u l=180n
M3529 nw480 t1281 vdd vdd pch w=2u l=180n
M3530 nw480 t1282 vdd vdd pch w=2u l=180n
CT1286 t1286 0 0.1f
M3531 nw480 t1281 t1286 0 nch w=1u l=180n
M3532 t1286 t1282 0 0 nch w=1u l=180n
Cnw480 nw480 0 2f
CT1287 t1287 0 0.1f
CT1288 t1288 0 0.1f
CT1289 t1289 0 0.1f
M3533 t1287 nw480 vdd vdd pch w=2u l=180n
M3534 t1287 nw479 vdd vdd pch w=2u l=180n
CT1290 t1290 0 0.1f
M3535 t1287 nw480 t1290 0 nch w=1u l=180n
M3536 t1290 nw479 0 0 nch w=1u l=180n
M3537 t1288 nw480 vdd vdd pch w=2u l=180n
M3538 t1288 t1287 vdd vdd pch w=2u l=180n
CT1291 t1291 0 0.1f
M3539 t1288 nw480 t1291 0 nch w=1u l=180n
M3540 t1291 t1287 0 0 nch w=1u l=180n
M3541 t1289 nw479 vdd vdd pch w=2u l=180n
M3542 t1289 t1287 vdd vdd pch w=2u l=180n
CT1292 t1292 0 0.1f
M3543 t1289 nw479 t1292 0 nch w=1u l=180n
M3544 t1292 t1287 0 0 nch w=1u l=180n
M3545 nw481 t1288 vdd vdd pch w=2u l=180n
M3546 nw481 t1289 vdd vdd pch w=2u l=180n
CT1293 t1293 0 0.1f
M3547 nw481 t1288 t1293 0 nch w=1u l=180n
M3548 t1293 t1289 0 0 nch w=1u l=180n
Cnw481 nw481 0 2f
M3549 nw482 nw64 vdd vdd pch w=2u l=180n
M3550 nw482 nw407 vdd vdd pch w=2u l=180n
CT1294 t1294 0 0.1f
M3551 nw482 nw64 t1294 0 nch w=1u l=180n
M3552 t1294 nw407 0 0 nch w=1u l=180n
Cnw482 nw482 0 2f
M3553 nw483 nw480 vdd vdd pch w=2u l=180n
M3554 nw483 nw479 vdd vdd pch w=2u l=180n
CT1295 t1295 0 0.1f
M3555 nw483 nw480 t1295 0 nch w=1u l=180n
M3556 t1295 nw479 0 0 nch w=1u l=180n
Cnw483 nw483 0 2f
M3557 nw484 nw482 vdd vdd pch w=2u l=180n
M3558 nw484 nw483 vdd vdd pch w=2u l=180n
CT1296 t1296 0 0.1f
M3559 nw484 nw482 t1296 0 nch w=1u l=180n
M3560 t1296 nw483 0 0 nch w=1u l=180n
Cnw484 nw484 0 2f
CT1297 t1297 0 0.1f
CT1298 t1298 0 0.1f
CT1299 t1299 0 0.1f
M3561 t1297 nw65 vdd vdd pch w=2u l=180n
M3562 t1297 nw411 vdd vdd pch w=2u l=180n
CT1300 t1300 0 0.1f
M3563 t1297 nw65 t1300 0 nch w=1u l=180n
M3564 t1300 nw411 0 0 nch w=1u l=180n
M3565 t1298 nw65 vdd vdd pch w=2u l=180n
M3566 t1298 t1297 vdd vdd pch w=2u l=180n
CT1301 t1301 0 0.1f
M3567 t1298 nw65 t1301 0 nch w=1u l=180n
M3568 t1301 t1297 0 0 nch w=1u l=180n
M3569 t1299 nw411 vdd vdd pch w=2u l=180n
M3570 t1299 t1297 vdd vdd pch w=2u l=180n
CT1302 t1302 0 0.1f
M3571 t1299 nw411 t1302 0 nch w=1u l=180n
M3572 t1302 t1297 0 0 nch w=1u l=180n
M3573 nw485 t1298 vdd vdd pch w=2u l=180n
M3574 nw485 t1299 vdd vdd pch w=2u l=180n
CT1303 t1303 0 0.1f
M3575 nw485 t1298 t1303 0 nch w=1u l=180n
M3576 t1303 t1299 0 0 nch w=1u l=180n
Cnw485 nw485 0 2f
CT1304 t1304 0 0.1f
M3577 t1304 nw65 vdd vdd pch w=2u l=180n
M3578 t1304 nw411 vdd vdd pch w=2u l=180n
CT1305 t1305 0 0.1f
M3579 t1304 nw65 t1305 0 nch w=1u l=180n
M3580 t1305 nw411 0 0 nch w=1u l=180n
M3581 nw486 t1304 vdd vdd pch w=2u l=180n
M3582 nw486 t1304 0 0 nch w=1u l=180n
Cnw486 nw486 0 2f
CT1306 t1306 0 0.1f
CT1307 t1307 0 0.1f
CT1308 t1308 0 0.1f
M3583 t1306 nw66 vdd vdd pch w=2u l=180n
M3584 t1306 nw416 vdd vdd pch w=2u l=180n
CT1309 t1309 0 0.1f
M3585 t1306 nw66 t1309 0 nch w=1u l=180n
M3586 t1309 nw416 0 0 nch w=1u l=180n
M3587 t1307 nw66 vdd vdd pch w=2u l=180n
M3588 t1307 t1306 vdd vdd pch w=2u l=180n
CT1310 t1310 0 0.1f
M3589 t1307 nw66 t1310 0 nch w=1u l=180n
M3590 t1310 t1306 0 0 nch w=1u l=180n
M3591 t1308 nw416 vdd vdd pch w=2u l=180n
M3592 t1308 t1306 vdd vdd pch w=2u l=180n
CT1311 t1311 0 0.1f
M3593 t1308 nw416 t1311 0 nch w=1u l=180n
M3594 t1311 t1306 0 0 nch w=1u l=180n
M3595 nw487 t1307 vdd vdd pch w=2u l=180n
M3596 nw487 t1308 vdd vdd pch w=2u l=180n
CT1312 t1312 0 0.1f
M3597 nw487 t1307 t1312 0 nch w=1u l=180n
M3598 t1312 t1308 0 0 nch w=1u l=180n
Cnw487 nw487 0 2f
CT1313 t1313 0 0.1f
CT1314 t1314 0 0.1f
CT1315 t1315 0 0.1f
M3599 t1313 nw487 vdd vdd pch w=2u l=180n
M3600 t1313 nw486 vdd vdd pch w=2u l=180n
CT1316 t1316 0 0.1f
M3601 t1313 nw487 t1316 0 nch w=1u l=180n
M3602 t1316 nw486 0 0 nch w=1u l=180n
M3603 t1314 nw487 vdd vdd pch w=2u l=180n
M3604 t1314 t1313 vdd vdd pch w=2u l=180n
CT1317 t1317 0 0.1f
M3605 t1314 nw487 t1317 0 nch w=1u l=180n
M3606 t1317 t1313 0 0 nch w=1u l=180n
M3607 t1315 nw486 vdd vdd pch w=2u l=180n
M3608 t1315 t1313 vdd vdd pch w=2u l=180n
CT1318 t1318 0 0.1f
M3609 t1315 nw486 t1318 0 nch w=1u l=180n
M3610 t1318 t1313 0 0 nch w=1u l=180n
M3611 nw488 t1314 vdd vdd pch w=2u l=180n
M3612 nw488 t1315 vdd vdd pch w=2u l=180n
CT1319 t1319 0 0.1f
M3613 nw488 t1314 t1319 0 nch w=1u l=180n
M3614 t1319 t1315 0 0 nch w=1u l=180n
Cnw488 nw488 0 2f
M3615 nw489 nw66 vdd vdd pch w=2u l=180n
M3616 nw489 nw416 vdd vdd pch w=2u l=180n
CT1320 t1320 0 0.1f
M3617 nw489 nw66 t1320 0 nch w=1u l=180n
M3618 t1320 nw416 0 0 nch w=1u l=180n
Cnw489 nw489 0 2f
M3619 nw490 nw487 vdd vdd pch w=2u l=180n
M3620 nw490 nw486 vdd vdd pch w=2u l=180n
CT1321 t1321 0 0.1f
M3621 nw490 nw487 t1321 0 nch w=1u l=180n
M3622 t1321 nw486 0 0 nch w=1u l=180n
Cnw490 nw490 0 2f
M3623 nw491 nw489 vdd vdd pch w=2u l=180n
M3624 nw491 nw490 vdd vdd pch w=2u l=180n
CT1322 t1322 0 0.1f
M3625 nw491 nw489 t1322 0 nch w=1u l=180n
M3626 t1322 nw490 0 0 nch w=1u l=180n
Cnw491 nw491 0 2f
CT1323 t1323 0 0.1f
CT1324 t1324 0 0.1f
CT1325 t1325 0 0.1f
M3627 t1323 nw67 vdd vdd pch w=2u l=180n
M3628 t1323 nw421 vdd vdd pch w=2u l=180n
CT1326 t1326 0 0.1f
M3629 t1323 nw67 t1326 0 nch w=1u l=180n
M3630 t1326 nw421 0 0 nch w=1u l=180n
M3631 t1324 nw67 vdd vdd pch w=2u l=180n
M3632 t1324 t1323 vdd vdd pch w=2u l=180n
CT1327 t1327 0 0.1f
M3633 t1324 nw67 t1327 0 nch w=1u l=180n
M3634 t1327 t1323 0 0 nch w=1u l=180n
M3635 t1325 nw421 vdd vdd pch w=2u l=180n
M3636 t1325 t1323 vdd vdd pch w=2u l=180n
CT1328 t1328 0 0.1f
M3637 t1325 nw421 t1328 0 nch w=1u l=180n
M3638 t1328 t1323 0 0 nch w=1u l=180n
M3639 nw492 t1324 vdd vdd pch w=2u l=180n
M3640 nw492 t1325 vdd vdd pch w=2u l=180n
CT1329 t1329 0 0.1f
M3641 nw492 t1324 t1329 0 nch w=1u l=180n
M3642 t1329 t1325 0 0 nch w=1u l=180n
Cnw492 nw492 0 2f
CT1330 t1330 0 0.1f
CT1331 t1331 0 0.1f
CT1332 t1332 0 0.1f
M3643 t1330 nw492 vdd vdd pch w=2u l=180n
M3644 t1330 nw491 vdd vdd pch w=2u l=180n
CT1333 t1333 0 0.1f
M3645 t1330 nw492 t1333 0 nch w=1u l=180n
M3646 t1333 nw491 0 0 nch w=1u l=180n
M3647 t1331 nw492 vdd vdd pch w=2u l=180n
M3648 t1331 t1330 vdd vdd pch w=2u l=180n
CT1334 t1334 0 0.1f
M3649 t1331 nw492 t1334 0 nch w=1u l=180n
M3650 t1334 t1330 0 0 nch w=1u l=180n
M3651 t1332 nw491 vdd vdd pch w=2u l=180n
M3652 t1332 t1330 vdd vdd pch w=2u l=180n
CT1335 t1335 0 0.1f
M3653 t1332 nw491 t1335 0 nch w=1u l=180n
M3654 t1335 t1330 0 0 nch w=1u l=180n
M3655 nw493 t1331 vdd vdd pch w=2u l=180n
M3656 nw493 t1332 vdd vdd pch w=2u l=180n
CT1336 t1336 0 0.1f
M3657 nw493 t1331 t1336 0 nch w=1u l=180n
M3658 t1336 t1332 0 0 nch w=1u l=180n
Cnw493 nw493 0 2f
M3659 nw494 nw67 vdd vdd pch w=2u l=180n
M3660 nw494 nw421 vdd vdd pch w=2u l=180n
CT1337 t1337 0 0.1f
M3661 nw494 nw67 t1337 0 nch w=1u l=180n
M3662 t1337 nw421 0 0 nch w=1u l=180n
Cnw494 nw494 0 2f
M3663 nw495 nw492 vdd vdd pch w=2u l=180n
M3664 nw495 nw491 vdd vdd pch w=2u l=180n
CT1338 t1338 0 0.1f
M3665 nw495 nw492 t1338 0 nch w=1u l=180n
M3666 t1338 nw491 0 0 nch w=1u l=180n
Cnw495 nw495 0 2f
M3667 nw496 nw494 vdd vdd pch w=2u l=180n
M3668 nw496 nw495 vdd vdd pch w=2u l=180n
CT1339 t1339 0 0.1f
M3669 nw496 nw494 t1339 0 nch w=1u l=180n
M3670 t1339 nw495 0 0 nch w=1u l=180n
Cnw496 nw496 0 2f
CT1340 t1340 0 0.1f
CT1341 t1341 0 0.1f
CT1342 t1342 0 0.1f
M3671 t1340 nw68 vdd vdd pch w=2u l=180n
M3672 t1340 nw426 vdd vdd pch w=2u l=180n
CT1343 t1343 0 0.1f
M3673 t1340 nw68 t1343 0 nch w=1u l=180n
M3674 t1343 nw426 0 0 nch w=1u l=180n
M3675 t1341 nw68 vdd vdd pch w=2u l=180n
M3676 t1341 t1340 vdd vdd pch w=2u l=180n
CT1344 t1344 0 0.1f
M3677 t1341 nw68 t1344 0 nch w=1u l=180n
M3678 t1344 t1340 0 0 nch w=1u l=180n
M3679 t1342 nw426 vdd vdd pch w=2u l=180n
M3680 t1342 t1340 vdd vdd pch w=2u l=180n
CT1345 t1345 0 0.1f
M3681 t1342 nw426 t1345 0 nch w=1u l=180n
M3682 t1345 t1340 0 0 nch w=1u l=180n
M3683 nw497 t1341 vdd vdd pch w=2u l=180n
M3684 nw497 t1342 vdd vdd pch w=2u l=180n
CT1346 t1346 0 0.1f
M3685 nw497 t1341 t1346 0 nch w=1u l=180n
M3686 t1346 t1342 0 0 nch w=1u l=180n
Cnw497 nw497 0 2f
CT1347 t1347 0 0.1f
CT1348 t1348 0 0.1f
CT1349 t1349 0 0.1f
M3687 t1347 nw497 vdd vdd pch w=2u l=180n
M3688 t1347 nw496 vdd vdd pch w=2u l=180n
CT1350 t1350 0 0.1f
M3689 t1347 nw497 t1350 0 nch w=1u l=180n
M3690 t1350 nw496 0 0 nch w=1u l=180n
M3691 t1348 nw497 vdd vdd pch w=2u l=180n
M3692 t1348 t1347 vdd vdd pch w=2u l=180n
CT1351 t1351 0 0.1f
M3693 t1348 nw497 t1351 0 nch w=1u l=180n
M3694 t1351 t1347 0 0 nch w=1u l=180n
M3695 t1349 nw496 vdd vdd pch w=2u l=180n
M3696 t1349 t1347 vdd vdd pch w=2u l=180n
CT1352 t1352 0 0.1f
M3697 t1349 nw496 t1352 0 nch w=1u l=180n
M3698 t1352 t1347 0 0 nch w=1u l=180n
M3699 nw498 t1348 vdd vdd pch w=2u l=180n
M3700 nw498 t1349 vdd vdd pch w=2u l=180n
CT1353 t1353 0 0.1f
M3701 nw498 t1348 t1353 0 nch w=1u l=180n
M3702 t1353 t1349 0 0 nch w=1u l=180n
Cnw498 nw498 0 2f
M3703 nw499 nw68 vdd vdd pch w=2u l=180n
M3704 nw499 nw426 vdd vdd pch w=2u l=180n
CT1354 t1354 0 0.1f
M3705 nw499 nw68 t1354 0 nch w=1u l=180n
M3706 t1354 nw426 0 0 nch w=1u l=180n
Cnw499 nw499 0 2f
M3707 nw500 nw497 vdd vdd pch w=2u l=180n
M3708 nw500 nw496 vdd vdd pch w=2u l=180n
CT1355 t1355 0 0.1f
M3709 nw500 nw497 t1355 0 nch w=1u l=180n
M3710 t1355 nw496 0 0 nch w=1u l=180n
Cnw500 nw500 0 2f
M3711 nw501 nw499 vdd vdd pch w=2u l=180n
M3712 nw501 nw500 vdd vdd pch w=2u l=180n
CT1356 t1356 0 0.1f
M3713 nw501 nw499 t1356 0 nch w=1u l=180n
M3714 t1356 nw500 0 0 nch w=1u l=180n
Cnw501 nw501 0 2f
CT1357 t1357 0 0.1f
CT1358 t1358 0 0.1f
CT1359 t1359 0 0.1f
M3715 t1357 nw69 vdd vdd pch w=2u l=180n
M3716 t1357 nw431 vdd vdd pch w=2u l=180n
CT1360 t1360 0 0.1f
M3717 t1357 nw69 t1360 0 nch w=1u l=180n
M3718 t1360 nw431 0 0 nch w=1u l=180n
M3719 t1358 nw69 vdd vdd pch w=2u l=180n
M3720 t1358 t1357 vdd vdd pch w=2u l=180n
CT1361 t1361 0 0.1f
M3721 t1358 nw69 t1361 0 nch w=1u l=180n
M3722 t1361 t1357 0 0 nch w=1u l=180n
M3723 t1359 nw431 vdd vdd pch w=2u l=180n
M3724 t1359 t1357 vdd vdd pch w=2u l=180n
CT1362 t1362 0 0.1f
M3725 t1359 nw431 t1362 0 nch w=1u l=180n
M3726 t1362 t1357 0 0 nch w=1u l=180n
M3727 nw502 t1358 vdd vdd pch w=2u l=180n
M3728 nw502 t1359 vdd vdd pch w=2u l=180n
CT1363 t1363 0 0.1f
M3729 nw502 t1358 t1363 0 nch w=1u l=180n
M3730 t1363 t1359 0 0 nch w=1u l=180n
Cnw502 nw502 0 2f
CT1364 t1364 0 0.1f
CT1365 t1365 0 0.1f
CT1366 t1366 0 0.1f
M3731 t1364 nw502 vdd vdd pch w=2u l=180n
M3732 t1364 nw501 vdd vdd pch w=2u l=180n
CT1367 t1367 0 0.1f
M3733 t1364 nw502 t1367 0 nch w=1u l=180n
M3734 t1367 nw501 0 0 nch w=1u l=180n
M3735 t1365 nw502 vdd vdd pch w=2u l=180n
M3736 t1365 t1364 vdd vdd pch w=2u l=180n
CT1368 t1368 0 0.1f
M3737 t1365 nw502 t1368 0 nch w=1u l=180n
M3738 t1368 t1364 0 0 nch w=1u l=180n
M3739 t1366 nw501 vdd vdd pch w=2u l=180n
M3740 t1366 t1364 vdd vdd pch w=2u l=180n
CT1369 t1369 0 0.1f
M3741 t1366 nw501 t1369 0 nch w=1u l=180n
M3742 t1369 t1364 0 0 nch w=1u l=180n
M3743 nw503 t1365 vdd vdd pch w=2u l=180n
M3744 nw503 t1366 vdd vdd pch w=2u l=180n
CT1370 t1370 0 0.1f
M3745 nw503 t1365 t1370 0 nch w=1u l=180n
M3746 t1370 t1366 0 0 nch w=1u l=180n
Cnw503 nw503 0 2f
M3747 nw504 nw69 vdd vdd pch w=2u l=180n
M3748 nw504 nw431 vdd vdd pch w=2u l=180n
CT1371 t1371 0 0.1f
M3749 nw504 nw69 t1371 0 nch w=1u l=180n
M3750 t1371 nw431 0 0 nch w=1u l=180n
Cnw504 nw504 0 2f
M3751 nw505 nw502 vdd vdd pch w=2u l=180n
M3752 nw505 nw501 vdd vdd pch w=2u l=180n
CT1372 t1372 0 0.1f
M3753 nw505 nw502 t1372 0 nch w=1u l=180n
M3754 t1372 nw501 0 0 nch w=1u l=180n
Cnw505 nw505 0 2f
M3755 nw506 nw504 vdd vdd pch w=2u l=180n
M3756 nw506 nw505 vdd vdd pch w=2u l=180n
CT1373 t1373 0 0.1f
M3757 nw506 nw504 t1373 0 nch w=1u l=180n
M3758 t1373 nw505 0 0 nch w=1u l=180n
Cnw506 nw506 0 2f
CT1374 t1374 0 0.1f
CT1375 t1375 0 0.1f
CT1376 t1376 0 0.1f
M3759 t1374 nw70 vdd vdd pch w=2u l=180n
M3760 t1374 nw436 vdd vdd pch w=2u l=180n
CT1377 t1377 0 0.1f
M3761 t1374 nw70 t1377 0 nch w=1u l=180n
M3762 t1377 nw436 0 0 nch w=1u l=180n
M3763 t1375 nw70 vdd vdd pch w=2u l=180n
M3764 t1375 t1374 vdd vdd pch w=2u l=180n
CT1378 t1378 0 0.1f
M3765 t1375 nw70 t1378 0 nch w=1u l=180n
M3766 t1378 t1374 0 0 nch w=1u l=180n
M3767 t1376 nw436 vdd vdd pch w=2u l=180n
M3768 t1376 t1374 vdd vdd pch w=2u l=180n
CT1379 t1379 0 0.1f
M3769 t1376 nw436 t1379 0 nch w=1u l=180n
M3770 t1379 t1374 0 0 nch w=1u l=180n
M3771 nw507 t1375 vdd vdd pch w=2u l=180n
M3772 nw507 t1376 vdd vdd pch w=2u l=180n
CT1380 t1380 0 0.1f
M3773 nw507 t1375 t1380 0 nch w=1u l=180n
M3774 t1380 t1376 0 0 nch w=1u l=180n
Cnw507 nw507 0 2f
CT1381 t1381 0 0.1f
CT1382 t1382 0 0.1f
CT1383 t1383 0 0.1f
M3775 t1381 nw507 vdd vdd pch w=2u l=180n
M3776 t1381 nw506 vdd vdd pch w=2u l=180n
CT1384 t1384 0 0.1f
M3777 t1381 nw507 t1384 0 nch w=1u l=180n
M3778 t1384 nw506 0 0 nch w=1u l=180n
M3779 t1382 nw507 vdd vdd pch w=2u l=180n
M3780 t1382 t1381 vdd vdd pch w=2u l=180n
CT1385 t1385 0 0.1f
M3781 t1382 nw507 t1385 0 nch w=1u l=180n
M3782 t1385 t1381 0 0 nch w=1u l=180n
M3783 t1383 nw506 vdd vdd pch w=2u l=180n
M3784 t1383 t1381 vdd vdd pch w=2u l=180n
CT1386 t1386 0 0.1f
M3785 t1383 nw506 t1386 0 nch w=1u l=180n
M3786 t1386 t1381 0 0 nch w=1u l=180n
M3787 nw508 t1382 vdd vdd pch w=2u l=180n
M3788 nw508 t1383 vdd vdd pch w=2u l=180n
CT1387 t1387 0 0.1f
M3789 nw508 t1382 t1387 0 nch w=1u l=180n
M3790 t1387 t1383 0 0 nch w=1u l=180n
Cnw508 nw508 0 2f
M3791 nw509 nw70 vdd vdd pch w=2u l=180n
M3792 nw509 nw436 vdd vdd pch w=2u l=180n
CT1388 t1388 0 0.1f
M3793 nw509 nw70 t1388 0 nch w=1u l=180n
M3794 t1388 nw436 0 0 nch w=1u l=180n
Cnw509 nw509 0 2f
M3795 nw510 nw507 vdd vdd pch w=2u l=180n
M3796 nw510 nw506 vdd vdd pch w=2u l=180n
CT1389 t1389 0 0.1f
M3797 nw510 nw507 t1389 0 nch w=1u l=180n
M3798 t1389 nw506 0 0 nch w=1u l=180n
Cnw510 nw510 0 2f
M3799 nw511 nw509 vdd vdd pch w=2u l=180n
M3800 nw511 nw510 vdd vdd pch w=2u l=180n
CT1390 t1390 0 0.1f
M3801 nw511 nw509 t1390 0 nch w=1u l=180n
M3802 t1390 nw510 0 0 nch w=1u l=180n
Cnw511 nw511 0 2f
CT1391 t1391 0 0.1f
CT1392 t1392 0 0.1f
CT1393 t1393 0 0.1f
M3803 t1391 nw71 vdd vdd pch w=2u l=180n
M3804 t1391 nw441 vdd vdd pch w=2u l=180n
CT1394 t1394 0 0.1f
M3805 t1391 nw71 t1394 0 nch w=1u l=180n
M3806 t1394 nw441 0 0 nch w=1u l=180n
M3807 t1392 nw71 vdd vdd pch w=2u l=180n
M3808 t1392 t1391 vdd vdd pch w=2u l=180n
CT1395 t1395 0 0.1f
M3809 t1392 nw71 t1395 0 nch w=1u l=180n
M3810 t1395 t1391 0 0 nch w=1u l=180n
M3811 t1393 nw441 vdd vdd pch w=2u l=180n
M3812 t1393 t1391 vdd vdd pch w=2u l=180n
CT1396 t1396 0 0.1f
M3813 t1393 nw441 t1396 0 nch w=1u l=180n
M3814 t1396 t1391 0 0 nch w=1u l=180n
M3815 nw512 t1392 vdd vdd pch w=2u l=180n
M3816 nw512 t1393 vdd vdd pch w=2u l=180n
CT1397 t1397 0 0.1f
M3817 nw512 t1392 t1397 0 nch w=1u l=180n
M3818 t1397 t1393 0 0 nch w=1u l=180n
Cnw512 nw512 0 2f
CT1398 t1398 0 0.1f
CT1399 t1399 0 0.1f
CT1400 t1400 0 0.1f
M3819 t1398 nw512 vdd vdd pch w=2u l=180n
M3820 t1398 nw511 vdd vdd pch w=2u l=180n
CT1401 t1401 0 0.1f
M3821 t1398 nw512 t1401 0 nch w=1u l=180n
M3822 t1401 nw511 0 0 nch w=1u l=180n
M3823 t1399 nw512 vdd vdd pch w=2u l=180n
M3824 t1399 t1398 vdd vdd pch w=2u l=180n
CT1402 t1402 0 0.1f
M3825 t1399 nw512 t1402 0 nch w=1u l=180n
M3826 t1402 t1398 0 0 nch w=1u l=180n
M3827 t1400 nw511 vdd vdd pch w=2u l=180n
M3828 t1400 t1398 vdd vdd pch w=2u l=180n
CT1403 t1403 0 0.1f
M3829 t1400 nw511 t1403 0 nch w=1u l=180n
M3830 t1403 t1398 0 0 nch w=1u l=180n
M3831 nw513 t1399 vdd vdd pch w=2u l=180n
M3832 nw513 t1400 vdd vdd pch w=2u l=180n
CT1404 t1404 0 0.1f
M3833 nw513 t1399 t1404 0 nch w=1u l=180n
M3834 t1404 t1400 0 0 nch w=1u l=180n
Cnw513 nw513 0 2f
M3835 nw514 nw71 vdd vdd pch w=2u l=180n
M3836 nw514 nw441 vdd vdd pch w=2u l=180n
CT1405 t1405 0 0.1f
M3837 nw514 nw71 t1405 0 nch w=1u l=180n
M3838 t1405 nw441 0 0 nch w=1u l=180n
Cnw514 nw514 0 2f
M3839 nw515 nw512 vdd vdd pch w=2u l=180n
M3840 nw515 nw511 vdd vdd pch w=2u l=180n
CT1406 t1406 0 0.1f
M3841 nw515 nw512 t1406 0 nch w=1u l=180n
M3842 t1406 nw511 0 0 nch w=1u l=180n
Cnw515 nw515 0 2f
M3843 nw516 nw514 vdd vdd pch w=2u l=180n
M3844 nw516 nw515 vdd vdd pch w=2u l=180n
CT1407 t1407 0 0.1f
M3845 nw516 nw514 t1407 0 nch w=1u l=180n
M3846 t1407 nw515 0 0 nch w=1u l=180n
Cnw516 nw516 0 2f
CT1408 t1408 0 0.1f
CT1409 t1409 0 0.1f
CT1410 t1410 0 0.1f
M3847 t1408 nw72 vdd vdd pch w=2u l=180n
M3848 t1408 nw446 vdd vdd pch w=2u l=180n
CT1411 t1411 0 0.1f
M3849 t1408 nw72 t1411 0 nch w=1u l=180n
M3850 t1411 nw446 0 0 nch w=1u l=180n
M3851 t1409 nw72 vdd vdd pch w=2u l=180n
M3852 t1409 t1408 vdd vdd pch w=2u l=180n
CT1412 t1412 0 0.1f
M3853 t1409 nw72 t1412 0 nch w=1u l=180n
M3854 t1412 t1408 0 0 nch w=1u l=180n
M3855 t1410 nw446 vdd vdd pch w=2u l=180n
M3856 t1410 t1408 vdd vdd pch w=2u l=180n
CT1413 t1413 0 0.1f
M3857 t1410 nw446 t1413 0 nch w=1u l=180n
M3858 t1413 t1408 0 0 nch w=1u l=180n
M3859 nw517 t1409 vdd vdd pch w=2u l=180n
M3860 nw517 t1410 vdd vdd pch w=2u l=180n
CT1414 t1414 0 0.1f
M3861 nw517 t1409 t1414 0 nch w=1u l=180n
M3862 t1414 t1410 0 0 nch w=1u l=180n
Cnw517 nw517 0 2f
CT1415 t1415 0 0.1f
CT1416 t1416 0 0.1f
CT1417 t1417 0 0.1f
M3863 t1415 nw517 vdd vdd pch w=2u l=180n
M3864 t1415 nw516 vdd vdd pch w=2u l=180n
CT1418 t1418 0 0.1f
M3865 t1415 nw517 t1418 0 nch w=1u l=180n
M3866 t1418 nw516 0 0 nch w=1u l=180n
M3867 t1416 nw517 vdd vdd pch w=2u l=180n
M3868 t1416 t1415 vdd vdd pch w=2u l=180n
CT1419 t1419 0 0.1f
M3869 t1416 nw517 t1419 0 nch w=1u l=180n
M3870 t1419 t1415 0 0 nch w=1u l=180n
M3871 t1417 nw516 vdd vdd pch w=2u l=180n
M3872 t1417 t1415 vdd vdd pch w=2u l=180n
CT1420 t1420 0 0.1f
M3873 t1417 nw516 t1420 0 nch w=1u l=180n
M3874 t1420 t1415 0 0 nch w=1u l=180n
M3875 nw518 t1416 vdd vdd pch w=2u l=180n
M3876 nw518 t1417 vdd vdd pch w=2u l=180n
CT1421 t1421 0 0.1f
M3877 nw518 t1416 t1421 0 nch w=1u l=180n
M3878 t1421 t1417 0 0 nch w=1u l=180n
Cnw518 nw518 0 2f
M3879 nw519 nw72 vdd vdd pch w=2u l=180n
M3880 nw519 nw446 vdd vdd pch w=2u l=180n
CT1422 t1422 0 0.1f
M3881 nw519 nw72 t1422 0 nch w=1u l=180n
M3882 t1422 nw446 0 0 nch w=1u l=180n
Cnw519 nw519 0 2f
M3883 nw520 nw517 vdd vdd pch w=2u l=180n
M3884 nw520 nw516 vdd vdd pch w=2u l=180n
CT1423 t1423 0 0.1f
M3885 nw520 nw517 t1423 0 nch w=1u l=180n
M3886 t1423 nw516 0 0 nch w=1u l=180n
Cnw520 nw520 0 2f
M3887 nw521 nw519 vdd vdd pch w=2u l=180n
M3888 nw521 nw520 vdd vdd pch w=2u l=180n
CT1424 t1424 0 0.1f
M3889 nw521 nw519 t1424 0 nch w=1u l=180n
M3890 t1424 nw520 0 0 nch w=1u l=180n
Cnw521 nw521 0 2f
CT1425 t1425 0 0.1f
CT1426 t1426 0 0.1f
CT1427 t1427 0 0.1f
M3891 t1425 nw73 vdd vdd pch w=2u l=180n
M3892 t1425 nw451 vdd vdd pch w=2u l=180n
CT1428 t1428 0 0.1f
M3893 t1425 nw73 t1428 0 nch w=1u l=180n
M3894 t1428 nw451 0 0 nch w=1u l=180n
M3895 t1426 nw73 vdd vdd pch w=2u l=180n
M3896 t1426 t1425 vdd vdd pch w=2u l=180n
CT1429 t1429 0 0.1f
M3897 t1426 nw73 t1429 0 nch w=1u l=180n
M3898 t1429 t1425 0 0 nch w=1u l=180n
M3899 t1427 nw451 vdd vdd pch w=2u l=180n
M3900 t1427 t1425 vdd vdd pch w=2u l=180n
CT1430 t1430 0 0.1f
M3901 t1427 nw451 t1430 0 nch w=1u l=180n
M3902 t1430 t1425 0 0 nch w=1u l=180n
M3903 nw522 t1426 vdd vdd pch w=2u l=180n
M3904 nw522 t1427 vdd vdd pch w=2u l=180n
CT1431 t1431 0 0.1f
M3905 nw522 t1426 t1431 0 nch w=1u l=180n
M3906 t1431 t1427 0 0 nch w=1u l=180n
Cnw522 nw522 0 2f
CT1432 t1432 0 0.1f
CT1433 t1433 0 0.1f
CT1434 t1434 0 0.1f
M3907 t1432 nw522 vdd vdd pch w=2u l=180n
M3908 t1432 nw521 vdd vdd pch w=2u l=180n
CT1435 t1435 0 0.1f
M3909 t1432 nw522 t1435 0 nch w=1u l=180n
M3910 t1435 nw521 0 0 nch w=1u l=180n
M3911 t1433 nw522 vdd vdd pch w=2u l=180n
M3912 t1433 t1432 vdd vdd pch w=2u l=180n
CT1436 t1436 0 0.1f
M3913 t1433 nw522 t1436 0 nch w=1u l=180n
M3914 t1436 t1432 0 0 nch w=1u l=180n
M3915 t1434 nw521 vdd vdd pch w=2u l=180n
M3916 t1434 t1432 vdd vdd pch w=2u l=180n
CT1437 t1437 0 0.1f
M3917 t1434 nw521 t1437 0 nch w=1u l=180n
M3918 t1437 t1432 0 0 nch w=1u l=180n
M3919 nw523 t1433 vdd vdd pch w=2u l=180n
M3920 nw523 t1434 vdd vdd pch w=2u l=180n
CT1438 t1438 0 0.1f
M3921 nw523 t1433 t1438 0 nch w=1u l=180n
M3922 t1438 t1434 0 0 nch w=1u l=180n
Cnw523 nw523 0 2f
M3923 nw524 nw73 vdd vdd pch w=2u l=180n
M3924 nw524 nw451 vdd vdd pch w=2u l=180n
CT1439 t1439 0 0.1f
M3925 nw524 nw73 t1439 0 nch w=1u l=180n
M3926 t1439 nw451 0 0 nch w=1u l=180n
Cnw524 nw524 0 2f
M3927 nw525 nw522 vdd vdd pch w=2u l=180n
M3928 nw525 nw521 vdd vdd pch w=2u l=180n
CT1440 t1440 0 0.1f
M3929 nw525 nw522 t1440 0 nch w=1u l=180n
M3930 t1440 nw521 0 0 nch w=1u l=180n
Cnw525 nw525 0 2f
M3931 nw526 nw524 vdd vdd pch w=2u l=180n
M3932 nw526 nw525 vdd vdd pch w=2u l=180n
CT1441 t1441 0 0.1f
M3933 nw526 nw524 t1441 0 nch w=1u l=180n
M3934 t1441 nw525 0 0 nch w=1u l=180n
Cnw526 nw526 0 2f
CT1442 t1442 0 0.1f
CT1443 t1443 0 0.1f
CT1444 t1444 0 0.1f
M3935 t1442 nw74 vdd vdd pch w=2u l=180n
M3936 t1442 nw456 vdd vdd pch w=2u l=180n
CT1445 t1445 0 0.1f
M3937 t1442 nw74 t1445 0 nch w=1u l=180n
M3938 t1445 nw456 0 0 nch w=1u l=180n
M3939 t1443 nw74 vdd vdd pch w=2u l=180n
M3940 t1443 t1442 vdd vdd pch w=2u l=180n
CT1446 t1446 0 0.1f
M3941 t1443 nw74 t1446 0 nch w=1u l=180n
M3942 t1446 t1442 0 0 nch w=1u l=180n
M3943 t1444 nw456 vdd vdd pch w=2u l=180n
M3944 t1444 t1442 vdd vdd pch w=2u l=180n
CT1447 t1447 0 0.1f
M3945 t1444 nw456 t1447 0 nch w=1u l=180n
M3946 t1447 t1442 0 0 nch w=1u l=180n
M3947 nw527 t1443 vdd vdd pch w=2u l=180n
M3948 nw527 t1444 vdd vdd pch w=2u l=180n
CT1448 t1448 0 0.1f
M3949 nw527 t1443 t1448 0 nch w=1u l=180n
M3950 t1448 t1444 0 0 nch w=1u l=180n
Cnw527 nw527 0 2f
CT1449 t1449 0 0.1f
CT1450 t1450 0 0.1f
CT1451 t1451 0 0.1f
M3951 t1449 nw527 vdd vdd pch w=2u l=180n
M3952 t1449 nw526 vdd vdd pch w=2u l=180n
CT1452 t1452 0 0.1f
M3953 t1449 nw527 t1452 0 nch w=1u l=180n
M3954 t1452 nw526 0 0 nch w=1u l=180n
M3955 t1450 nw527 vdd vdd pch w=2u l=180n
M3956 t1450 t1449 vdd vdd pch w=2u l=180n
CT1453 t1453 0 0.1f
M3957 t1450 nw527 t1453 0 nch w=1u l=180n
M3958 t1453 t1449 0 0 nch w=1u l=180n
M3959 t1451 nw526 vdd vdd pch w=2u l=180n
M3960 t1451 t1449 vdd vdd pch w=2u l=180n
CT1454 t1454 0 0.1f
M3961 t1451 nw526 t1454 0 nch w=1u l=180n
M3962 t1454 t1449 0 0 nch w=1u l=180n
M3963 nw528 t1450 vdd vdd pch w=2u l=180n
M3964 nw528 t1451 vdd vdd pch w=2u l=180n
CT1455 t1455 0 0.1f
M3965 nw528 t1450 t1455 0 nch w=1u l=180n
M3966 t1455 t1451 0 0 nch w=1u l=180n
Cnw528 nw528 0 2f
M3967 nw529 nw74 vdd vdd pch w=2u l=180n
M3968 nw529 nw456 vdd vdd pch w=2u l=180n
CT1456 t1456 0 0.1f
M3969 nw529 nw74 t1456 0 nch w=1u l=180n
M3970 t1456 nw456 0 0 nch w=1u l=180n
Cnw529 nw529 0 2f
M3971 nw530 nw527 vdd vdd pch w=2u l=180n
M3972 nw530 nw526 vdd vdd pch w=2u l=180n
CT1457 t1457 0 0.1f
M3973 nw530 nw527 t1457 0 nch w=1u l=180n
M3974 t1457 nw526 0 0 nch w=1u l=180n
Cnw530 nw530 0 2f
M3975 nw531 nw529 vdd vdd pch w=2u l=180n
M3976 nw531 nw530 vdd vdd pch w=2u l=180n
CT1458 t1458 0 0.1f
M3977 nw531 nw529 t1458 0 nch w=1u l=180n
M3978 t1458 nw530 0 0 nch w=1u l=180n
Cnw531 nw531 0 2f
CT1459 t1459 0 0.1f
CT1460 t1460 0 0.1f
CT1461 t1461 0 0.1f
M3979 t1459 nw75 vdd vdd pch w=2u l=180n
M3980 t1459 nw461 vdd vdd pch w=2u l=180n
CT1462 t1462 0 0.1f
M3981 t1459 nw75 t1462 0 nch w=1u l=180n
M3982 t1462 nw461 0 0 nch w=1u l=180n
M3983 t1460 nw75 vdd vdd pch w=2u l=180n
M3984 t1460 t1459 vdd vdd pch w=2u l=180n
CT1463 t1463 0 0.1f
M3985 t1460 nw75 t1463 0 nch w=1u l=180n
M3986 t1463 t1459 0 0 nch w=1u l=180n
M3987 t1461 nw461 vdd vdd pch w=2u l=180n
M3988 t1461 t1459 vdd vdd pch w=2u l=180n
CT1464 t1464 0 0.1f
M3989 t1461 nw461 t1464 0 nch w=1u l=180n
M3990 t1464 t1459 0 0 nch w=1u l=180n
M3991 nw532 t1460 vdd vdd pch w=2u l=180n
M3992 nw532 t1461 vdd vdd pch w=2u l=180n
CT1465 t1465 0 0.1f
M3993 nw532 t1460 t1465 0 nch w=1u l=180n
M3994 t1465 t1461 0 0 nch w=1u l=180n
Cnw532 nw532 0 2f
CT1466 t1466 0 0.1f
CT1467 t1467 0 0.1f
CT1468 t1468 0 0.1f
M3995 t1466 nw532 vdd vdd pch w=2u l=180n
M3996 t1466 nw531 vdd vdd pch w=2u l=180n
CT1469 t1469 0 0.1f
M3997 t1466 nw532 t1469 0 nch w=1u l=180n
M3998 t1469 nw531 0 0 nch w=1u l=180n
M3999 t1467 nw532 vdd vdd pch w=2u l=180n
M4000 t1467 t1466 vdd vdd pch w=2u l=180n
CT1470 t1470 0 0.1f
M4001 t1467 nw532 t1470 0 nch w=1u l=180n
M4002 t1470 t1466 0 0 nch w=1u l=180n
M4003 t1468 nw531 vdd vdd pch w=2u l=180n
M4004 t1468 t1466 vdd vdd pch w=2u l=180n
CT1471 t1471 0 0.1f
M4005 t1468 nw531 t1471 0 nch w=1u l=180n
M4006 t1471 t1466 0 0 nch w=1u l=180n
M4007 nw533 t1467 vdd vdd pch w=2u l=180n
M4008 nw533 t1468 vdd vdd pch w=2u l=180n
CT1472 t1472 0 0.1f
M4009 nw533 t1467 t1472 0 nch w=1u l=180n
M4010 t1472 t1468 0 0 nch w=1u l=180n
Cnw533 nw533 0 2f
M4011 nw534 nw75 vdd vdd pch w=2u l=180n
M4012 nw534 nw461 vdd vdd pch w=2u l=180n
CT1473 t1473 0 0.1f
M4013 nw534 nw75 t1473 0 nch w=1u l=180n
M4014 t1473 nw461 0 0 nch w=1u l=180n
Cnw534 nw534 0 2f
M4015 nw535 nw532 vdd vdd pch w=2u l=180n
M4016 nw535 nw531 vdd vdd pch w=2u l=180n
CT1474 t1474 0 0.1f
M4017 nw535 nw532 t1474 0 nch w=1u l=180n
M4018 t1474 nw531 0 0 nch w=1u l=180n
Cnw535 nw535 0 2f
M4019 nw536 nw534 vdd vdd pch w=2u l=180n
M4020 nw536 nw535 vdd vdd pch w=2u l=180n
CT1475 t1475 0 0.1f
M4021 nw536 nw534 t1475 0 nch w=1u l=180n
M4022 t1475 nw535 0 0 nch w=1u l=180n
Cnw536 nw536 0 2f
CT1476 t1476 0 0.1f
CT1477 t1477 0 0.1f
CT1478 t1478 0 0.1f
M4023 t1476 nw76 vdd vdd pch w=2u l=180n
M4024 t1476 nw466 vdd vdd pch w=2u l=180n
CT1479 t1479 0 0.1f
M4025 t1476 nw76 t1479 0 nch w=1u l=180n
M4026 t1479 nw466 0 0 nch w=1u l=180n
M4027 t1477 nw76 vdd vdd pch w=2u l=180n
M4028 t1477 t1476 vdd vdd pch w=2u l=180n
CT1480 t1480 0 0.1f
M4029 t1477 nw76 t1480 0 nch w=1u l=180n
M4030 t1480 t1476 0 0 nch w=1u l=180n
M4031 t1478 nw466 vdd vdd pch w=2u l=180n
M4032 t1478 t1476 vdd vdd pch w=2u l=180n
CT1481 t1481 0 0.1f
M4033 t1478 nw466 t1481 0 nch w=1u l=180n
M4034 t1481 t1476 0 0 nch w=1u l=180n
M4035 nw537 t1477 vdd vdd pch w=2u l=180n
M4036 nw537 t1478 vdd vdd pch w=2u l=180n
CT1482 t1482 0 0.1f
M4037 nw537 t1477 t1482 0 nch w=1u l=180n
M4038 t1482 t1478 0 0 nch w=1u l=180n
Cnw537 nw537 0 2f
CT1483 t1483 0 0.1f
CT1484 t1484 0 0.1f
CT1485 t1485 0 0.1f
M4039 t1483 nw537 vdd vdd pch w=2u l=180n
M4040 t1483 nw536 vdd vdd pch w=2u l=180n
CT1486 t1486 0 0.1f
M4041 t1483 nw537 t1486 0 nch w=1u l=180n
M4042 t1486 nw536 0 0 nch w=1u l=180n
M4043 t1484 nw537 vdd vdd pch w=2u l=180n
M4044 t1484 t1483 vdd vdd pch w=2u l=180n
CT1487 t1487 0 0.1f
M4045 t1484 nw537 t1487 0 nch w=1u l=180n
M4046 t1487 t1483 0 0 nch w=1u l=180n
M4047 t1485 nw536 vdd vdd pch w=2u l=180n
M4048 t1485 t1483 vdd vdd pch w=2u l=180n
CT1488 t1488 0 0.1f
M4049 t1485 nw536 t1488 0 nch w=1u l=180n
M4050 t1488 t1483 0 0 nch w=1u l=180n
M4051 nw538 t1484 vdd vdd pch w=2u l=180n
M4052 nw538 t1485 vdd vdd pch w=2u l=180n
CT1489 t1489 0 0.1f
M4053 nw538 t1484 t1489 0 nch w=1u l=180n
M4054 t1489 t1485 0 0 nch w=1u l=180n
Cnw538 nw538 0 2f
M4055 nw539 nw76 vdd vdd pch w=2u l=180n
M4056 nw539 nw466 vdd vdd pch w=2u l=180n
CT1490 t1490 0 0.1f
M4057 nw539 nw76 t1490 0 nch w=1u l=180n
M4058 t1490 nw466 0 0 nch w=1u l=180n
Cnw539 nw539 0 2f
M4059 nw540 nw537 vdd vdd pch w=2u l=180n
M4060 nw540 nw536 vdd vdd pch w=2u l=180n
CT1491 t1491 0 0.1f
M4061 nw540 nw537 t1491 0 nch w=1u l=180n
M4062 t1491 nw536 0 0 nch w=1u l=180n
Cnw540 nw540 0 2f
M4063 nw541 nw539 vdd vdd pch w=2u l=180n
M4064 nw541 nw540 vdd vdd pch w=2u l=180n
CT1492 t1492 0 0.1f
M4065 nw541 nw539 t1492 0 nch w=1u l=180n
M4066 t1492 nw540 0 0 nch w=1u l=180n
Cnw541 nw541 0 2f
CT1493 t1493 0 0.1f
CT1494 t1494 0 0.1f
CT1495 t1495 0 0.1f
M4067 t1493 nw77 vdd vdd pch w=2u l=180n
M4068 t1493 nw471 vdd vdd pch w=2u l=180n
CT1496 t1496 0 0.1f
M4069 t1493 nw77 t1496 0 nch w=1u l=180n
M4070 t1496 nw471 0 0 nch w=1u l=180n
M4071 t1494 nw77 vdd vdd pch w=2u l=180n
M4072 t1494 t1493 vdd vdd pch w=2u l=180n
CT1497 t1497 0 0.1f
M4073 t1494 nw77 t1497 0 nch w=1u l=180n
M4074 t1497 t1493 0 0 nch w=1u l=180n
M4075 t1495 nw471 vdd vdd pch w=2u l=180n
M4076 t1495 t1493 vdd vdd pch w=2u l=180n
CT1498 t1498 0 0.1f
M4077 t1495 nw471 t1498 0 nch w=1u l=180n
M4078 t1498 t1493 0 0 nch w=1u l=180n
M4079 nw542 t1494 vdd vdd pch w=2u l=180n
M4080 nw542 t1495 vdd vdd pch w=2u l=180n
CT1499 t1499 0 0.1f
M4081 nw542 t1494 t1499 0 nch w=1u l=180n
M4082 t1499 t1495 0 0 nch w=1u l=180n
Cnw542 nw542 0 2f
CT1500 t1500 0 0.1f
CT1501 t1501 0 0.1f
CT1502 t1502 0 0.1f
M4083 t1500 nw542 vdd vdd pch w=2u l=180n
M4084 t1500 nw541 vdd vdd pch w=2u l=180n
CT1503 t1503 0 0.1f
M4085 t1500 nw542 t1503 0 nch w=1u l=180n
M4086 t1503 nw541 0 0 nch w=1u l=180n
M4087 t1501 nw542 vdd vdd pch w=2u l=180n
M4088 t1501 t1500 vdd vdd pch w=2u l=180n
CT1504 t1504 0 0.1f
M4089 t1501 nw542 t1504 0 nch w=1u l=180n
M4090 t1504 t1500 0 0 nch w=1u l=180n
M4091 t1502 nw541 vdd vdd pch w=2u l=180n
M4092 t1502 t1500 vdd vdd pch w=2u l=180n
CT1505 t1505 0 0.1f
M4093 t1502 nw541 t1505 0 nch w=1u l=180n
M4094 t1505 t1500 0 0 nch w=1u l=180n
M4095 nw543 t1501 vdd vdd pch w=2u l=180n
M4096 nw543 t1502 vdd vdd pch w=2u l=180n
CT1506 t1506 0 0.1f
M4097 nw543 t1501 t1506 0 nch w=1u l=180n
M4098 t1506 t1502 0 0 nch w=1u l=180n
Cnw543 nw543 0 2f
M4099 nw544 nw77 vdd vdd pch w=2u l=180n
M4100 nw544 nw471 vdd vdd pch w=2u l=180n
CT1507 t1507 0 0.1f
M4101 nw544 nw77 t1507 0 nch w=1u l=180n
M4102 t1507 nw471 0 0 nch w=1u l=180n
Cnw544 nw544 0 2f
M4103 nw545 nw542 vdd vdd pch w=2u l=180n
M4104 nw545 nw541 vdd vdd pch w=2u l=180n
CT1508 t1508 0 0.1f
M4105 nw545 nw542 t1508 0 nch w=1u l=180n
M4106 t1508 nw541 0 0 nch w=1u l=180n
Cnw545 nw545 0 2f
M4107 nw546 nw544 vdd vdd pch w=2u l=180n
M4108 nw546 nw545 vdd vdd pch w=2u l=180n
CT1509 t1509 0 0.1f
M4109 nw546 nw544 t1509 0 nch w=1u l=180n
M4110 t1509 nw545 0 0 nch w=1u l=180n
Cnw546 nw546 0 2f
CT1510 t1510 0 0.1f
CT1511 t1511 0 0.1f
CT1512 t1512 0 0.1f
M4111 t1510 nw78 vdd vdd pch w=2u l=180n
M4112 t1510 nw476 vdd vdd pch w=2u l=180n
CT1513 t1513 0 0.1f
M4113 t1510 nw78 t1513 0 nch w=1u l=180n
M4114 t1513 nw476 0 0 nch w=1u l=180n
M4115 t1511 nw78 vdd vdd pch w=2u l=180n
M4116 t1511 t1510 vdd vdd pch w=2u l=180n
CT1514 t1514 0 0.1f
M4117 t1511 nw78 t1514 0 nch w=1u l=180n
M4118 t1514 t1510 0 0 nch w=1u l=180n
M4119 t1512 nw476 vdd vdd pch w=2u l=180n
M4120 t1512 t1510 vdd vdd pch w=2u l=180n
CT1515 t1515 0 0.1f
M4121 t1512 nw476 t1515 0 nch w=1u l=180n
M4122 t1515 t1510 0 0 nch w=1u l=180n
M4123 nw547 t1511 vdd vdd pch w=2u l=180n
M4124 nw547 t1512 vdd vdd pch w=2u l=180n
CT1516 t1516 0 0.1f
M4125 nw547 t1511 t1516 0 nch w=1u l=180n
M4126 t1516 t1512 0 0 nch w=1u l=180n
Cnw547 nw547 0 2f
CT1517 t1517 0 0.1f
CT1518 t1518 0 0.1f
CT1519 t1519 0 0.1f
M4127 t1517 nw547 vdd vdd pch w=2u l=180n
M4128 t1517 nw546 vdd vdd pch w=2u l=180n
CT1520 t1520 0 0.1f
M4129 t1517 nw547 t1520 0 nch w=1u l=180n
M4130 t1520 nw546 0 0 nch w=1u l=180n
M4131 t1518 nw547 vdd vdd pch w=2u l=180n
M4132 t1518 t1517 vdd vdd pch w=2u l=180n
CT1521 t1521 0 0.1f
M4133 t1518 nw547 t1521 0 nch w=1u l=180n
M4134 t1521 t1517 0 0 nch w=1u l=180n
M4135 t1519 nw546 vdd vdd pch w=2u l=180n
M4136 t1519 t1517 vdd vdd pch w=2u l=180n
CT1522 t1522 0 0.1f
M4137 t1519 nw546 t1522 0 nch w=1u l=180n
M4138 t1522 t1517 0 0 nch w=1u l=180n
M4139 nw548 t1518 vdd vdd pch w=2u l=180n
M4140 nw548 t1519 vdd vdd pch w=2u l=180n
CT1523 t1523 0 0.1f
M4141 nw548 t1518 t1523 0 nch w=1u l=180n
M4142 t1523 t1519 0 0 nch w=1u l=180n
Cnw548 nw548 0 2f
M4143 nw549 nw78 vdd vdd pch w=2u l=180n
M4144 nw549 nw476 vdd vdd pch w=2u l=180n
CT1524 t1524 0 0.1f
M4145 nw549 nw78 t1524 0 nch w=1u l=180n
M4146 t1524 nw476 0 0 nch w=1u l=180n
Cnw549 nw549 0 2f
M4147 nw550 nw547 vdd vdd pch w=2u l=180n
M4148 nw550 nw546 vdd vdd pch w=2u l=180n
CT1525 t1525 0 0.1f
M4149 nw550 nw547 t1525 0 nch w=1u l=180n
M4150 t1525 nw546 0 0 nch w=1u l=180n
Cnw550 nw550 0 2f
M4151 nw551 nw549 vdd vdd pch w=2u l=180n
M4152 nw551 nw550 vdd vdd pch w=2u l=180n
CT1526 t1526 0 0.1f
M4153 nw551 nw549 t1526 0 nch w=1u l=180n
M4154 t1526 nw550 0 0 nch w=1u l=180n
Cnw551 nw551 0 2f
CT1527 t1527 0 0.1f
CT1528 t1528 0 0.1f
CT1529 t1529 0 0.1f
M4155 t1527 nw79 vdd vdd pch w=2u l=180n
M4156 t1527 nw481 vdd vdd pch w=2u l=180n
CT1530 t1530 0 0.1f
M4157 t1527 nw79 t1530 0 nch w=1u l=180n
M4158 t1530 nw481 0 0 nch w=1u l=180n
M4159 t1528 nw79 vdd vdd pch w=2u l=180n
M4160 t1528 t1527 vdd vdd pch w=2u l=180n
CT1531 t1531 0 0.1f
M4161 t1528 nw79 t1531 0 nch w=1u l=180n
M4162 t1531 t1527 0 0 nch w=1u l=180n
M4163 t1529 nw481 vdd vdd pch w=2u l=180n
M4164 t1529 t1527 vdd vdd pch w=2u l=180n
CT1532 t1532 0 0.1f
M4165 t1529 nw481 t1532 0 nch w=1u l=180n
M4166 t1532 t1527 0 0 nch w=1u l=180n
M4167 nw552 t1528 vdd vdd pch w=2u l=180n
M4168 nw552 t1529 vdd vdd pch w=2u l=180n
CT1533 t1533 0 0.1f
M4169 nw552 t1528 t1533 0 nch w=1u l=180n
M4170 t1533 t1529 0 0 nch w=1u l=180n
Cnw552 nw552 0 2f
CT1534 t1534 0 0.1f
CT1535 t1535 0 0.1f
CT1536 t1536 0 0.1f
M4171 t1534 nw552 vdd vdd pch w=2u l=180n
M4172 t1534 nw551 vdd vdd pch w=2u l=180n
CT1537 t1537 0 0.1f
M4173 t1534 nw552 t1537 0 nch w=1u l=180n
M4174 t1537 nw551 0 0 nch w=1u l=180n
M4175 t1535 nw552 vdd vdd pch w=2u l=180n
M4176 t1535 t1534 vdd vdd pch w=2u l=180n
CT1538 t1538 0 0.1f
M4177 t1535 nw552 t1538 0 nch w=1u l=180n
M4178 t1538 t1534 0 0 nch w=1u l=180n
M4179 t1536 nw551 vdd vdd pch w=2u l=180n
M4180 t1536 t1534 vdd vdd pch w=2u l=180n
CT1539 t1539 0 0.1f
M4181 t1536 nw551 t1539 0 nch w=1u l=180n
M4182 t1539 t1534 0 0 nch w=1u l=180n
M4183 nw553 t1535 vdd vdd pch w=2u l=180n
M4184 nw553 t1536 vdd vdd pch w=2u l=180n
CT1540 t1540 0 0.1f
M4185 nw553 t1535 t1540 0 nch w=1u l=180n
M4186 t1540 t1536 0 0 nch w=1u l=180n
Cnw553 nw553 0 2f
M4187 nw554 nw79 vdd vdd pch w=2u l=180n
M4188 nw554 nw481 vdd vdd pch w=2u l=180n
CT1541 t1541 0 0.1f
M4189 nw554 nw79 t1541 0 nch w=1u l=180n
M4190 t1541 nw481 0 0 nch w=1u l=180n
Cnw554 nw554 0 2f
M4191 nw555 nw552 vdd vdd pch w=2u l=180n
M4192 nw555 nw551 vdd vdd pch w=2u l=180n
CT1542 t1542 0 0.1f
M4193 nw555 nw552 t1542 0 nch w=1u l=180n
M4194 t1542 nw551 0 0 nch w=1u l=180n
Cnw555 nw555 0 2f
M4195 nw556 nw554 vdd vdd pch w=2u l=180n
M4196 nw556 nw555 vdd vdd pch w=2u l=180n
CT1543 t1543 0 0.1f
M4197 nw556 nw554 t1543 0 nch w=1u l=180n
M4198 t1543 nw555 0 0 nch w=1u l=180n
Cnw556 nw556 0 2f
CT1544 t1544 0 0.1f
CT1545 t1545 0 0.1f
CT1546 t1546 0 0.1f
M4199 t1544 nw80 vdd vdd pch w=2u l=180n
M4200 t1544 nw484 vdd vdd pch w=2u l=180n
CT1547 t1547 0 0.1f
M4201 t1544 nw80 t1547 0 nch w=1u l=180n
M4202 t1547 nw484 0 0 nch w=1u l=180n
M4203 t1545 nw80 vdd vdd pch w=2u l=180n
M4204 t1545 t1544 vdd vdd pch w=2u l=180n
CT1548 t1548 0 0.1f
M4205 t1545 nw80 t1548 0 nch w=1u l=180n
M4206 t1548 t1544 0 0 nch w=1u l=180n
M4207 t1546 nw484 vdd vdd pch w=2u l=180n
M4208 t1546 t1544 vdd vdd pch w=2u l=180n
CT1549 t1549 0 0.1f
M4209 t1546 nw484 t1549 0 nch w=1u l=180n
M4210 t1549 t1544 0 0 nch w=1u l=180n
M4211 nw557 t1545 vdd vdd pch w=2u l=180n
M4212 nw557 t1546 vdd vdd pch w=2u l=180n
CT1550 t1550 0 0.1f
M4213 nw557 t1545 t1550 0 nch w=1u l=180n
M4214 t1550 t1546 0 0 nch w=1u l=180n
Cnw557 nw557 0 2f
CT1551 t1551 0 0.1f
CT1552 t1552 0 0.1f
CT1553 t1553 0 0.1f
M4215 t1551 nw557 vdd vdd pch w=2u l=180n
M4216 t1551 nw556 vdd vdd pch w=2u l=180n
CT1554 t1554 0 0.1f
M4217 t1551 nw557 t1554 0 nch w=1u l=180n
M4218 t1554 nw556 0 0 nch w=1u l=180n
M4219 t1552 nw557 vdd vdd pch w=2u l=180n
M4220 t1552 t1551 vdd vdd pch w=2u l=180n
CT1555 t1555 0 0.1f
M4221 t1552 nw557 t1555 0 nch w=1u l=180n
M4222 t1555 t1551 0 0 nch w=1u l=180n
M4223 t1553 nw556 vdd vdd pch w=2u l=180n
M4224 t1553 t1551 vdd vdd pch w=2u l=180n
CT1556 t1556 0 0.1f
M4225 t1553 nw556 t1556 0 nch w=1u l=180n
M4226 t1556 t1551 0 0 nch w=1u l=180n
M4227 nw558 t1552 vdd vdd pch w=2u l=180n
M4228 nw558 t1553 vdd vdd pch w=2u l=180n
CT1557 t1557 0 0.1f
M4229 nw558 t1552 t1557 0 nch w=1u l=180n
M4230 t1557 t1553 0 0 nch w=1u l=180n
Cnw558 nw558 0 2f
M4231 nw559 nw80 vdd vdd pch w=2u l=180n
M4232 nw559 nw484 vdd vdd pch w=2u l=180n
CT1558 t1558 0 0.1f
M4233 nw559 nw80 t1558 0 nch w=1u l=180n
M4234 t1558 nw484 0 0 nch w=1u l=180n
Cnw559 nw559 0 2f
M4235 nw560 nw557 vdd vdd pch w=2u l=180n
M4236 nw560 nw556 vdd vdd pch w=2u l=180n
CT1559 t1559 0 0.1f
M4237 nw560 nw557 t1559 0 nch w=1u l=180n
M4238 t1559 nw556 0 0 nch w=1u l=180n
Cnw560 nw560 0 2f
M4239 nw561 nw559 vdd vdd pch w=2u l=180n
M4240 nw561 nw560 vdd vdd pch w=2u l=180n
CT1560 t1560 0 0.1f
M4241 nw561 nw559 t1560 0 nch w=1u l=180n
M4242 t1560 nw560 0 0 nch w=1u l=180n
Cnw561 nw561 0 2f
CT1561 t1561 0 0.1f
CT1562 t1562 0 0.1f
CT1563 t1563 0 0.1f
M4243 t1561 nw81 vdd vdd pch w=2u l=180n
M4244 t1561 nw488 vdd vdd pch w=2u l=180n
CT1564 t1564 0 0.1f
M4245 t1561 nw81 t1564 0 nch w=1u l=180n
M4246 t1564 nw488 0 0 nch w=1u l=180n
M4247 t1562 nw81 vdd vdd pch w=2u l=180n
M4248 t1562 t1561 vdd vdd pch w=2u l=180n
CT1565 t1565 0 0.1f
M4249 t1562 nw81 t1565 0 nch w=1u l=180n
M4250 t1565 t1561 0 0 nch w=1u l=180n
M4251 t1563 nw488 vdd vdd pch w=2u l=180n
M4252 t1563 t1561 vdd vdd pch w=2u l=180n
CT1566 t1566 0 0.1f
M4253 t1563 nw488 t1566 0 nch w=1u l=180n
M4254 t1566 t1561 0 0 nch w=1u l=180n
M4255 nw562 t1562 vdd vdd pch w=2u l=180n
M4256 nw562 t1563 vdd vdd pch w=2u l=180n
CT1567 t1567 0 0.1f
M4257 nw562 t1562 t1567 0 nch w=1u l=180n
M4258 t1567 t1563 0 0 nch w=1u l=180n
Cnw562 nw562 0 2f
CT1568 t1568 0 0.1f
M4259 t1568 nw81 vdd vdd pch w=2u l=180n
M4260 t1568 nw488 vdd vdd pch w=2u l=180n
CT1569 t1569 0 0.1f
M4261 t1568 nw81 t1569 0 nch w=1u l=180n
M4262 t1569 nw488 0 0 nch w=1u l=180n
M4263 nw563 t1568 vdd vdd pch w=2u l=180n
M4264 nw563 t1568 0 0 nch w=1u l=180n
Cnw563 nw563 0 2f
CT1570 t1570 0 0.1f
CT1571 t1571 0 0.1f
CT1572 t1572 0 0.1f
M4265 t1570 nw82 vdd vdd pch w=2u l=180n
M4266 t1570 nw493 vdd vdd pch w=2u l=180n
CT1573 t1573 0 0.1f
M4267 t1570 nw82 t1573 0 nch w=1u l=180n
M4268 t1573 nw493 0 0 nch w=1u l=180n
M4269 t1571 nw82 vdd vdd pch w=2u l=180n
M4270 t1571 t1570 vdd vdd pch w=2u l=180n
CT1574 t1574 0 0.1f
M4271 t1571 nw82 t1574 0 nch w=1u l=180n
M4272 t1574 t1570 0 0 nch w=1u l=180n
M4273 t1572 nw493 vdd vdd pch w=2u l=180n
M4274 t1572 t1570 vdd vdd pch w=2u l=180n
CT1575 t1575 0 0.1f
M4275 t1572 nw493 t1575 0 nch w=1u l=180n
M4276 t1575 t1570 0 0 nch w=1u l=180n
M4277 nw564 t1571 vdd vdd pch w=2u l=180n
M4278 nw564 t1572 vdd vdd pch w=2u l=180n
CT1576 t1576 0 0.1f
M4279 nw564 t1571 t1576 0 nch w=1u l=180n
M4280 t1576 t1572 0 0 nch w=1u l=180n
Cnw564 nw564 0 2f
CT1577 t1577 0 0.1f
CT1578 t1578 0 0.1f
CT1579 t1579 0 0.1f
M4281 t1577 nw564 vdd vdd pch w=2u l=180n
M4282 t1577 nw563 vdd vdd pch w=2u l=180n
CT1580 t1580 0 0.1f
M4283 t1577 nw564 t1580 0 nch w=1u l=180n
M4284 t1580 nw563 0 0 nch w=1u l=180n
M4285 t1578 nw564 vdd vdd pch w=2u l=180n
M4286 t1578 t1577 vdd vdd pch w=2u l=180n
CT1581 t1581 0 0.1f
M4287 t1578 nw564 t1581 0 nch w=1u l=180n
M4288 t1581 t1577 0 0 nch w=1u l=180n
M4289 t1579 nw563 vdd vdd pch w=2u l=180n
M4290 t1579 t1577 vdd vdd pch w=2u l=180n
CT1582 t1582 0 0.1f
M4291 t1579 nw563 t1582 0 nch w=1u l=180n
M4292 t1582 t1577 0 0 nch w=1u l=180n
M4293 nw565 t1578 vdd vdd pch w=2u l=180n
M4294 nw565 t1579 vdd vdd pch w=2u l=180n
CT1583 t1583 0 0.1f
M4295 nw565 t1578 t1583 0 nch w=1u l=180n
M4296 t1583 t1579 0 0 nch w=1u l=180n
Cnw565 nw565 0 2f
M4297 nw566 nw82 vdd vdd pch w=2u l=180n
M4298 nw566 nw493 vdd vdd pch w=2u l=180n
CT1584 t1584 0 0.1f
M4299 nw566 nw82 t1584 0 nch w=1u l=180n
M4300 t1584 nw493 0 0 nch w=1u l=180n
Cnw566 nw566 0 2f
M4301 nw567 nw564 vdd vdd pch w=2u l=180n
M4302 nw567 nw563 vdd vdd pch w=2u l=180n
CT1585 t1585 0 0.1f
M4303 nw567 nw564 t1585 0 nch w=1u l=180n
M4304 t1585 nw563 0 0 nch w=1u l=180n
Cnw567 nw567 0 2f
M4305 nw568 nw566 vdd vdd pch w=2u l=180n
M4306 nw568 nw567 vdd vdd pch w=2u l=180n
CT1586 t1586 0 0.1f
M4307 nw568 nw566 t1586 0 nch w=1u l=180n
M4308 t1586 nw567 0 0 nch w=1u l=180n
Cnw568 nw568 0 2f
CT1587 t1587 0 0.1f
CT1588 t1588 0 0.1f
CT1589 t1589 0 0.1f
M4309 t1587 nw83 vdd vdd pch w=2u l=180n
M4310 t1587 nw498 vdd vdd pch w=2u l=180n
CT1590 t1590 0 0.1f
M4311 t1587 nw83 t1590 0 nch w=1u l=180n
M4312 t1590 nw498 0 0 nch w=1u l=180n
M4313 t1588 nw83 vdd vdd pch w=2u l=180n
M4314 t1588 t1587 vdd vdd pch w=2u l=180n
CT1591 t1591 0 0.1f
M4315 t1588 nw83 t1591 0 nch w=1u l=180n
M4316 t1591 t1587 0 0 nch w=1u l=180n
M4317 t1589 nw498 vdd vdd pch w=2u l=180n
M4318 t1589 t1587 vdd vdd pch w=2u l=180n
CT1592 t1592 0 0.1f
M4319 t1589 nw498 t1592 0 nch w=1u l=180n
M4320 t1592 t1587 0 0 nch w=1u l=180n
M4321 nw569 t1588 vdd vdd pch w=2u l=180n
M4322 nw569 t1589 vdd vdd pch w=2u l=180n
CT1593 t1593 0 0.1f
M4323 nw569 t1588 t1593 0 nch w=1u l=180n
M4324 t1593 t1589 0 0 nch w=1u l=180n
Cnw569 nw569 0 2f
CT1594 t1594 0 0.1f
CT1595 t1595 0 0.1f
CT1596 t1596 0 0.1f
M4325 t1594 nw569 vdd vdd pch w=2u l=180n
M4326 t1594 nw568 vdd vdd pch w=2u l=180n
CT1597 t1597 0 0.1f
M4327 t1594 nw569 t1597 0 nch w=1u l=180n
M4328 t1597 nw568 0 0 nch w=1u l=180n
M4329 t1595 nw569 vdd vdd pch w=2u l=180n
M4330 t1595 t1594 vdd vdd pch w=2u l=180n
CT1598 t1598 0 0.1f
M4331 t1595 nw569 t1598 0 nch w=1u l=180n
M4332 t1598 t1594 0 0 nch w=1u l=180n
M4333 t1596 nw568 vdd vdd pch w=2u l=180n
M4334 t1596 t1594 vdd vdd pch w=2u l=180n
CT1599 t1599 0 0.1f
M4335 t1596 nw568 t1599 0 nch w=1u l=180n
M4336 t1599 t1594 0 0 nch w=1u l=180n
M4337 nw570 t1595 vdd vdd pch w=2u l=180n
M4338 nw570 t1596 vdd vdd pch w=2u l=180n
CT1600 t1600 0 0.1f
M4339 nw570 t1595 t1600 0 nch w=1u l=180n
M4340 t1600 t1596 0 0 nch w=1u l=180n
Cnw570 nw570 0 2f
M4341 nw571 nw83 vdd vdd pch w=2u l=180n
M4342 nw571 nw498 vdd vdd pch w=2u l=180n
CT1601 t1601 0 0.1f
M4343 nw571 nw83 t1601 0 nch w=1u l=180n
M4344 t1601 nw498 0 0 nch w=1u l=180n
Cnw571 nw571 0 2f
M4345 nw572 nw569 vdd vdd pch w=2u l=180n
M4346 nw572 nw568 vdd vdd pch w=2u l=180n
CT1602 t1602 0 0.1f
M4347 nw572 nw569 t1602 0 nch w=1u l=180n
M4348 t1602 nw568 0 0 nch w=1u l=180n
Cnw572 nw572 0 2f
M4349 nw573 nw571 vdd vdd pch w=2u l=180n
M4350 nw573 nw572 vdd vdd pch w=2u l=180n
CT1603 t1603 0 0.1f
M4351 nw573 nw571 t1603 0 nch w=1u l=180n
M4352 t1603 nw572 0 0 nch w=1u l=180n
Cnw573 nw573 0 2f
CT1604 t1604 0 0.1f
CT1605 t1605 0 0.1f
CT1606 t1606 0 0.1f
M4353 t1604 nw84 vdd vdd pch w=2u l=180n
M4354 t1604 nw503 vdd vdd pch w=2u l=180n
CT1607 t1607 0 0.1f
M4355 t1604 nw84 t1607 0 nch w=1u l=180n
M4356 t1607 nw503 0 0 nch w=1u l=180n
M4357 t1605 nw84 vdd vdd pch w=2u l=180n
M4358 t1605 t1604 vdd vdd pch w=2u l=180n
CT1608 t1608 0 0.1f
M4359 t1605 nw84 t1608 0 nch w=1u l=180n
M4360 t1608 t1604 0 0 nch w=1u l=180n
M4361 t1606 nw503 vdd vdd pch w=2u l=180n
M4362 t1606 t1604 vdd vdd pch w=2u l=180n
CT1609 t1609 0 0.1f
M4363 t1606 nw503 t1609 0 nch w=1u l=180n
M4364 t1609 t1604 0 0 nch w=1u l=180n
M4365 nw574 t1605 vdd vdd pch w=2u l=180n
M4366 nw574 t1606 vdd vdd pch w=2u l=180n
CT1610 t1610 0 0.1f
M4367 nw574 t1605 t1610 0 nch w=1u l=180n
M4368 t1610 t1606 0 0 nch w=1u l=180n
Cnw574 nw574 0 2f
CT1611 t1611 0 0.1f
CT1612 t1612 0 0.1f
CT1613 t1613 0 0.1f
M4369 t1611 nw574 vdd vdd pch w=2u l=180n
M4370 t1611 nw573 vdd vdd pch w=2u l=180n
CT1614 t1614 0 0.1f
M4371 t1611 nw574 t1614 0 nch w=1u l=180n
M4372 t1614 nw573 0 0 nch w=1u l=180n
M4373 t1612 nw574 vdd vdd pch w=2u l=180n
M4374 t1612 t1611 vdd vdd pch w=2u l=180n
CT1615 t1615 0 0.1f
M4375 t1612 nw574 t1615 0 nch w=1u l=180n
M4376 t1615 t1611 0 0 nch w=1u l=180n
M4377 t1613 nw573 vdd vdd pch w=2u l=180n
M4378 t1613 t1611 vdd vdd pch w=2u l=180n
CT1616 t1616 0 0.1f
M4379 t1613 nw573 t1616 0 nch w=1u l=180n
M4380 t1616 t1611 0 0 nch w=1u l=180n
M4381 nw575 t1612 vdd vdd pch w=2u l=180n
M4382 nw575 t1613 vdd vdd pch w=2u l=180n
CT1617 t1617 0 0.1f
M4383 nw575 t1612 t1617 0 nch w=1u l=180n
M4384 t1617 t1613 0 0 nch w=1u l=180n
Cnw575 nw575 0 2f
M4385 nw576 nw84 vdd vdd pch w=2u l=180n
M4386 nw576 nw503 vdd vdd pch w=2u l=180n
CT1618 t1618 0 0.1f
M4387 nw576 nw84 t1618 0 nch w=1u l=180n
M4388 t1618 nw503 0 0 nch w=1u l=180n
Cnw576 nw576 0 2f
M4389 nw577 nw574 vdd vdd pch w=2u l=180n
M4390 nw577 nw573 vdd vdd pch w=2u l=180n
CT1619 t1619 0 0.1f
M4391 nw577 nw574 t1619 0 nch w=1u l=180n
M4392 t1619 nw573 0 0 nch w=1u l=180n
Cnw577 nw577 0 2f
M4393 nw578 nw576 vdd vdd pch w=2u l=180n
M4394 nw578 nw577 vdd vdd pch w=2u l=180n
CT1620 t1620 0 0.1f
M4395 nw578 nw576 t1620 0 nch w=1u l=180n
M4396 t1620 nw577 0 0 nch w=1u l=180n
Cnw578 nw578 0 2f
CT1621 t1621 0 0.1f
CT1622 t1622 0 0.1f
CT1623 t1623 0 0.1f
M4397 t1621 nw85 vdd vdd pch w=2u l=180n
M4398 t1621 nw508 vdd vdd pch w=2u l=180n
CT1624 t1624 0 0.1f
M4399 t1621 nw85 t1624 0 nch w=1u l=180n
M4400 t1624 nw508 0 0 nch w=1u l=180n
M4401 t1622 nw85 vdd vdd pch w=2u l=180n
M4402 t1622 t1621 vdd vdd pch w=2u l=180n
CT1625 t1625 0 0.1f
M4403 t1622 nw85 t1625 0 nch w=1u l=180n
M4404 t1625 t1621 0 0 nch w=1u l=180n
M4405 t1623 nw508 vdd vdd pch w=2u l=180n
M4406 t1623 t1621 vdd vdd pch w=2u l=180n
CT1626 t1626 0 0.1f
M4407 t1623 nw508 t1626 0 nch w=1u l=180n
M4408 t1626 t1621 0 0 nch w=1u l=180n
M4409 nw579 t1622 vdd vdd pch w=2u l=180n
M4410 nw579 t1623 vdd vdd pch w=2u l=180n
CT1627 t1627 0 0.1f
M4411 nw579 t1622 t1627 0 nch w=1u l=180n
M4412 t1627 t1623 0 0 nch w=1u l=180n
Cnw579 nw579 0 2f
CT1628 t1628 0 0.1f
CT1629 t1629 0 0.1f
CT1630 t1630 0 0.1f
M4413 t1628 nw579 vdd vdd pch w=2u l=180n
M4414 t1628 nw578 vdd vdd pch w=2u l=180n
CT1631 t1631 0 0.1f
M4415 t1628 nw579 t1631 0 nch w=1u l=180n
M4416 t1631 nw578 0 0 nch w=1u l=180n
M4417 t1629 nw579 vdd vdd pch w=2u l=180n
M4418 t1629 t1628 vdd vdd pch w=2u l=180n
CT1632 t1632 0 0.1f
M4419 t1629 nw579 t1632 0 nch w=1u l=180n
M4420 t1632 t1628 0 0 nch w=1u l=180n
M4421 t1630 nw578 vdd vdd pch w=2u l=180n
M4422 t1630 t1628 vdd vdd pch w=2u l=180n
CT1633 t1633 0 0.1f
M4423 t1630 nw578 t1633 0 nch w=1u l=180n
M4424 t1633 t1628 0 0 nch w=1u l=180n
M4425 nw580 t1629 vdd vdd pch w=2u l=180n
M4426 nw580 t1630 vdd vdd pch w=2u l=180n
CT1634 t1634 0 0.1f
M4427 nw580 t1629 t1634 0 nch w=1u l=180n
M4428 t1634 t1630 0 0 nch w=1u l=180n
Cnw580 nw580 0 2f
M4429 nw581 nw85 vdd vdd pch w=2u l=180n
M4430 nw581 nw508 vdd vdd pch w=2u l=180n
CT1635 t1635 0 0.1f
M4431 nw581 nw85 t1635 0 nch w=1u l=180n
M4432 t1635 nw508 0 0 nch w=1u l=180n
Cnw581 nw581 0 2f
M4433 nw582 nw579 vdd vdd pch w=2u l=180n
M4434 nw582 nw578 vdd vdd pch w=2u l=180n
CT1636 t1636 0 0.1f
M4435 nw582 nw579 t1636 0 nch w=1u l=180n
M4436 t1636 nw578 0 0 nch w=1u l=180n
Cnw582 nw582 0 2f
M4437 nw583 nw581 vdd vdd pch w=2u l=180n
M4438 nw583 nw582 vdd vdd pch w=2u l=180n
CT1637 t1637 0 0.1f
M4439 nw583 nw581 t1637 0 nch w=1u l=180n
M4440 t1637 nw582 0 0 nch w=1u l=180n
Cnw583 nw583 0 2f
CT1638 t1638 0 0.1f
CT1639 t1639 0 0.1f
CT1640 t1640 0 0.1f
M4441 t1638 nw86 vdd vdd pch w=2u l=180n
M4442 t1638 nw513 vdd vdd pch w=2u l=180n
CT1641 t1641 0 0.1f
M4443 t1638 nw86 t1641 0 nch w=1u l=180n
M4444 t1641 nw513 0 0 nch w=1u l=180n
M4445 t1639 nw86 vdd vdd pch w=2u l=180n
M4446 t1639 t1638 vdd vdd pch w=2u l=180n
CT1642 t1642 0 0.1f
M4447 t1639 nw86 t1642 0 nch w=1u l=180n
M4448 t1642 t1638 0 0 nch w=1u l=180n
M4449 t1640 nw513 vdd vdd pch w=2u l=180n
M4450 t1640 t1638 vdd vdd pch w=2u l=180n
CT1643 t1643 0 0.1f
M4451 t1640 nw513 t1643 0 nch w=1u l=180n
M4452 t1643 t1638 0 0 nch w=1u l=180n
M4453 nw584 t1639 vdd vdd pch w=2u l=180n
M4454 nw584 t1640 vdd vdd pch w=2u l=180n
CT1644 t1644 0 0.1f
M4455 nw584 t1639 t1644 0 nch w=1u l=180n
M4456 t1644 t1640 0 0 nch w=1u l=180n
Cnw584 nw584 0 2f
CT1645 t1645 0 0.1f
CT1646 t1646 0 0.1f
CT1647 t1647 0 0.1f
M4457 t1645 nw584 vdd vdd pch w=2u l=180n
M4458 t1645 nw583 vdd vdd pch w=2u l=180n
CT1648 t1648 0 0.1f
M4459 t1645 nw584 t1648 0 nch w=1u l=180n
M4460 t1648 nw583 0 0 nch w=1u l=180n
M4461 t1646 nw584 vdd vdd pch w=2u l=180n
M4462 t1646 t1645 vdd vdd pch w=2u l=180n
CT1649 t1649 0 0.1f
M4463 t1646 nw584 t1649 0 nch w=1u l=180n
M4464 t1649 t1645 0 0 nch w=1u l=180n
M4465 t1647 nw583 vdd vdd pch w=2u l=180n
M4466 t1647 t1645 vdd vdd pch w=2u l=180n
CT1650 t1650 0 0.1f
M4467 t1647 nw583 t1650 0 nch w=1u l=180n
M4468 t1650 t1645 0 0 nch w=1u l=180n
M4469 nw585 t1646 vdd vdd pch w=2u l=180n
M4470 nw585 t1647 vdd vdd pch w=2u l=180n
CT1651 t1651 0 0.1f
M4471 nw585 t1646 t1651 0 nch w=1u l=180n
M4472 t1651 t1647 0 0 nch w=1u l=180n
Cnw585 nw585 0 2f
M4473 nw586 nw86 vdd vdd pch w=2u l=180n
M4474 nw586 nw513 vdd vdd pch w=2u l=180n
CT1652 t1652 0 0.1f
M4475 nw586 nw86 t1652 0 nch w=1u l=180n
M4476 t1652 nw513 0 0 nch w=1u l=180n
Cnw586 nw586 0 2f
M4477 nw587 nw584 vdd vdd pch w=2u l=180n
M4478 nw587 nw583 vdd vdd pch w=2u l=180n
CT1653 t1653 0 0.1f
M4479 nw587 nw584 t1653 0 nch w=1u l=180n
M4480 t1653 nw583 0 0 nch w=1u l=180n
Cnw587 nw587 0 2f
M4481 nw588 nw586 vdd vdd pch w=2u l=180n
M4482 nw588 nw587 vdd vdd pch w=2u l=180n
CT1654 t1654 0 0.1f
M4483 nw588 nw586 t1654 0 nch w=1u l=180n
M4484 t1654 nw587 0 0 nch w=1u l=180n
Cnw588 nw588 0 2f
CT1655 t1655 0 0.1f
CT1656 t1656 0 0.1f
CT1657 t1657 0 0.1f
M4485 t1655 nw87 vdd vdd pch w=2u l=180n
M4486 t1655 nw518 vdd vdd pch w=2u l=180n
CT1658 t1658 0 0.1f
M4487 t1655 nw87 t1658 0 nch w=1u l=180n
M4488 t1658 nw518 0 0 nch w=1u l=180n
M4489 t1656 nw87 vdd vdd pch w=2u l=180n
M4490 t1656 t1655 vdd vdd pch w=2u l=180n
CT1659 t1659 0 0.1f
M4491 t1656 nw87 t1659 0 nch w=1u l=180n
M4492 t1659 t1655 0 0 nch w=1u l=180n
M4493 t1657 nw518 vdd vdd pch w=2u l=180n
M4494 t1657 t1655 vdd vdd pch w=2u l=180n
CT1660 t1660 0 0.1f
M4495 t1657 nw518 t1660 0 nch w=1u l=180n
M4496 t1660 t1655 0 0 nch w=1u l=180n
M4497 nw589 t1656 vdd vdd pch w=2u l=180n
M4498 nw589 t1657 vdd vdd pch w=2u l=180n
CT1661 t1661 0 0.1f
M4499 nw589 t1656 t1661 0 nch w=1u l=180n
M4500 t1661 t1657 0 0 nch w=1u l=180n
Cnw589 nw589 0 2f
CT1662 t1662 0 0.1f
CT1663 t1663 0 0.1f
CT1664 t1664 0 0.1f
M4501 t1662 nw589 vdd vdd pch w=2u l=180n
M4502 t1662 nw588 vdd vdd pch w=2u l=180n
CT1665 t1665 0 0.1f
M4503 t1662 nw589 t1665 0 nch w=1u l=180n
M4504 t1665 nw588 0 0 nch w=1u l=180n
M4505 t1663 nw589 vdd vdd pch w=2u l=180n
M4506 t1663 t1662 vdd vdd pch w=2u l=180n
CT1666 t1666 0 0.1f
M4507 t1663 nw589 t1666 0 nch w=1u l=180n
M4508 t1666 t1662 0 0 nch w=1u l=180n
M4509 t1664 nw588 vdd vdd pch w=2u l=180n
M4510 t1664 t1662 vdd vdd pch w=2u l=180n
CT1667 t1667 0 0.1f
M4511 t1664 nw588 t1667 0 nch w=1u l=180n
M4512 t1667 t1662 0 0 nch w=1u l=180n
M4513 nw590 t1663 vdd vdd pch w=2u l=180n
M4514 nw590 t1664 vdd vdd pch w=2u l=180n
CT1668 t1668 0 0.1f
M4515 nw590 t1663 t1668 0 nch w=1u l=180n
M4516 t1668 t1664 0 0 nch w=1u l=180n
Cnw590 nw590 0 2f
M4517 nw591 nw87 vdd vdd pch w=2u l=180n
M4518 nw591 nw518 vdd vdd pch w=2u l=180n
CT1669 t1669 0 0.1f
M4519 nw591 nw87 t1669 0 nch w=1u l=180n
M4520 t1669 nw518 0 0 nch w=1u l=180n
Cnw591 nw591 0 2f
M4521 nw592 nw589 vdd vdd pch w=2u l=180n
M4522 nw592 nw588 vdd vdd pch w=2u l=180n
CT1670 t1670 0 0.1f
M4523 nw592 nw589 t1670 0 nch w=1u l=180n
M4524 t1670 nw588 0 0 nch w=1u l=180n
Cnw592 nw592 0 2f
M4525 nw593 nw591 vdd vdd pch w=2u l=180n
M4526 nw593 nw592 vdd vdd pch w=2u l=180n
CT1671 t1671 0 0.1f
M4527 nw593 nw591 t1671 0 nch w=1u l=180n
M4528 t1671 nw592 0 0 nch w=1u l=180n
Cnw593 nw593 0 2f
CT1672 t1672 0 0.1f
CT1673 t1673 0 0.1f
CT1674 t1674 0 0.1f
M4529 t1672 nw88 vdd vdd pch w=2u l=180n
M4530 t1672 nw523 vdd vdd pch w=2u l=180n
CT1675 t1675 0 0.1f
M4531 t1672 nw88 t1675 0 nch w=1u l=180n
M4532 t1675 nw523 0 0 nch w=1u l=180n
M4533 t1673 nw88 vdd vdd pch w=2u l=180n
M4534 t1673 t1672 vdd vdd pch w=2u l=180n
CT1676 t1676 0 0.1f
M4535 t1673 nw88 t1676 0 nch w=1u l=180n
M4536 t1676 t1672 0 0 nch w=1u l=180n
M4537 t1674 nw523 vdd vdd pch w=2u l=180n
M4538 t1674 t1672 vdd vdd pch w=2u l=180n
CT1677 t1677 0 0.1f
M4539 t1674 nw523 t1677 0 nch w=1u l=180n
M4540 t1677 t1672 0 0 nch w=1u l=180n
M4541 nw594 t1673 vdd vdd pch w=2u l=180n
M4542 nw594 t1674 vdd vdd pch w=2u l=180n
CT1678 t1678 0 0.1f
M4543 nw594 t1673 t1678 0 nch w=1u l=180n
M4544 t1678 t1674 0 0 nch w=1u l=180n
Cnw594 nw594 0 2f
CT1679 t1679 0 0.1f
CT1680 t1680 0 0.1f
CT1681 t1681 0 0.1f
M4545 t1679 nw594 vdd vdd pch w=2u l=180n
M4546 t1679 nw593 vdd vdd pch w=2u l=180n
CT1682 t1682 0 0.1f
M4547 t1679 nw594 t1682 0 nch w=1u l=180n
M4548 t1682 nw593 0 0 nch w=1u l=180n
M4549 t1680 nw594 vdd vdd pch w=2u l=180n
M4550 t1680 t1679 vdd vdd pch w=2u l=180n
CT1683 t1683 0 0.1f
M4551 t1680 nw594 t1683 0 nch w=1u l=180n
M4552 t1683 t1679 0 0 nch w=1u l=180n
M4553 t1681 nw593 vdd vdd pch w=2u l=180n
M4554 t1681 t1679 vdd vdd pch w=2u l=180n
CT1684 t1684 0 0.1f
M4555 t1681 nw593 t1684 0 nch w=1u l=180n
M4556 t1684 t1679 0 0 nch w=1u l=180n
M4557 nw595 t1680 vdd vdd pch w=2u l=180n
M4558 nw595 t1681 vdd vdd pch w=2u l=180n
CT1685 t1685 0 0.1f
M4559 nw595 t1680 t1685 0 nch w=1u l=180n
M4560 t1685 t1681 0 0 nch w=1u l=180n
Cnw595 nw595 0 2f
M4561 nw596 nw88 vdd vdd pch w=2u l=180n
M4562 nw596 nw523 vdd vdd pch w=2u l=180n
CT1686 t1686 0 0.1f
M4563 nw596 nw88 t1686 0 nch w=1u l=180n
M4564 t1686 nw523 0 0 nch w=1u l=180n
Cnw596 nw596 0 2f
M4565 nw597 nw594 vdd vdd pch w=2u l=180n
M4566 nw597 nw593 vdd vdd pch w=2u l=180n
CT1687 t1687 0 0.1f
M4567 nw597 nw594 t1687 0 nch w=1u l=180n
M4568 t1687 nw593 0 0 nch w=1u l=180n
Cnw597 nw597 0 2f
M4569 nw598 nw596 vdd vdd pch w=2u l=180n
M4570 nw598 nw597 vdd vdd pch w=2u l=180n
CT1688 t1688 0 0.1f
M4571 nw598 nw596 t1688 0 nch w=1u l=180n
M4572 t1688 nw597 0 0 nch w=1u l=180n
Cnw598 nw598 0 2f
CT1689 t1689 0 0.1f
CT1690 t1690 0 0.1f
CT1691 t1691 0 0.1f
M4573 t1689 nw89 vdd vdd pch w=2u l=180n
M4574 t1689 nw528 vdd vdd pch w=2u l=180n
CT1692 t1692 0 0.1f
M4575 t1689 nw89 t1692 0 nch w=1u l=180n
M4576 t1692 nw528 0 0 nch w=1u l=180n
M4577 t1690 nw89 vdd vdd pch w=2u l=180n
M4578 t1690 t1689 vdd vdd pch w=2u l=180n
CT1693 t1693 0 0.1f
M4579 t1690 nw89 t1693 0 nch w=1u l=180n
M4580 t1693 t1689 0 0 nch w=1u l=180n
M4581 t1691 nw528 vdd vdd pch w=2u l=180n
M4582 t1691 t1689 vdd vdd pch w=2u l=180n
CT1694 t1694 0 0.1f
M4583 t1691 nw528 t1694 0 nch w=1u l=180n
M4584 t1694 t1689 0 0 nch w=1u l=180n
M4585 nw599 t1690 vdd vdd pch w=2u l=180n
M4586 nw599 t1691 vdd vdd pch w=2u l=180n
CT1695 t1695 0 0.1f
M4587 nw599 t1690 t1695 0 nch w=1u l=180n
M4588 t1695 t1691 0 0 nch w=1u l=180n
Cnw599 nw599 0 2f
CT1696 t1696 0 0.1f
CT1697 t1697 0 0.1f
CT1698 t1698 0 0.1f
M4589 t1696 nw599 vdd vdd pch w=2u l=180n
M4590 t1696 nw598 vdd vdd pch w=2u l=180n
CT1699 t1699 0 0.1f
M4591 t1696 nw599 t1699 0 nch w=1u l=180n
M4592 t1699 nw598 0 0 nch w=1u l=180n
M4593 t1697 nw599 vdd vdd pch w=2u l=180n
M4594 t1697 t1696 vdd vdd pch w=2u l=180n
CT1700 t1700 0 0.1f
M4595 t1697 nw599 t1700 0 nch w=1u l=180n
M4596 t1700 t1696 0 0 nch w=1u l=180n
M4597 t1698 nw598 vdd vdd pch w=2u l=180n
M4598 t1698 t1696 vdd vdd pch w=2u l=180n
CT1701 t1701 0 0.1f
M4599 t1698 nw598 t1701 0 nch w=1u l=180n
M4600 t1701 t1696 0 0 nch w=1u l=180n
M4601 nw600 t1697 vdd vdd pch w=2u l=180n
M4602 nw600 t1698 vdd vdd pch w=2u l=180n
CT1702 t1702 0 0.1f
M4603 nw600 t1697 t1702 0 nch w=1u l=180n
M4604 t1702 t1698 0 0 nch w=1u l=180n
Cnw600 nw600 0 2f
M4605 nw601 nw89 vdd vdd pch w=2u l=180n
M4606 nw601 nw528 vdd vdd pch w=2u l=180n
CT1703 t1703 0 0.1f
M4607 nw601 nw89 t1703 0 nch w=1u l=180n
M4608 t1703 nw528 0 0 nch w=1u l=180n
Cnw601 nw601 0 2f
M4609 nw602 nw599 vdd vdd pch w=2u l=180n
M4610 nw602 nw598 vdd vdd pch w=2u l=180n
CT1704 t1704 0 0.1f
M4611 nw602 nw599 t1704 0 nch w=1u l=180n
M4612 t1704 nw598 0 0 nch w=1u l=180n
Cnw602 nw602 0 2f
M4613 nw603 nw601 vdd vdd pch w=2u l=180n
M4614 nw603 nw602 vdd vdd pch w=2u l=180n
CT1705 t1705 0 0.1f
M4615 nw603 nw601 t1705 0 nch w=1u l=180n
M4616 t1705 nw602 0 0 nch w=1u l=180n
Cnw603 nw603 0 2f
CT1706 t1706 0 0.1f
CT1707 t1707 0 0.1f
CT1708 t1708 0 0.1f
M4617 t1706 nw90 vdd vdd pch w=2u l=180n
M4618 t1706 nw533 vdd vdd pch w=2u l=180n
CT1709 t1709 0 0.1f
M4619 t1706 nw90 t1709 0 nch w=1u l=180n
M4620 t1709 nw533 0 0 nch w=1u l=180n
M4621 t1707 nw90 vdd vdd pch w=2u l=180n
M4622 t1707 t1706 vdd vdd pch w=2u l=180n
CT1710 t1710 0 0.1f
M4623 t1707 nw90 t1710 0 nch w=1u l=180n
M4624 t1710 t1706 0 0 nch w=1u l=180n
M4625 t1708 nw533 vdd vdd pch w=2u l=180n
M4626 t1708 t1706 vdd vdd pch w=2u l=180n
CT1711 t1711 0 0.1f
M4627 t1708 nw533 t1711 0 nch w=1u l=180n
M4628 t1711 t1706 0 0 nch w=1u l=180n
M4629 nw604 t1707 vdd vdd pch w=2u l=180n
M4630 nw604 t1708 vdd vdd pch w=2u l=180n
CT1712 t1712 0 0.1f
M4631 nw604 t1707 t1712 0 nch w=1u l=180n
M4632 t1712 t1708 0 0 nch w=1u l=180n
Cnw604 nw604 0 2f
CT1713 t1713 0 0.1f
CT1714 t1714 0 0.1f
CT1715 t1715 0 0.1f
M4633 t1713 nw604 vdd vdd pch w=2u l=180n
M4634 t1713 nw603 vdd vdd pch w=2u l=180n
CT1716 t1716 0 0.1f
M4635 t1713 nw604 t1716 0 nch w=1u l=180n
M4636 t1716 nw603 0 0 nch w=1u l=180n
M4637 t1714 nw604 vdd vdd pch w=2u l=180n
M4638 t1714 t1713 vdd vdd pch w=2u l=180n
CT1717 t1717 0 0.1f
M4639 t1714 nw604 t1717 0 nch w=1u l=180n
M4640 t1717 t1713 0 0 nch w=1u l=180n
M4641 t1715 nw603 vdd vdd pch w=2u l=180n
M4642 t1715 t1713 vdd vdd pch w=2u l=180n
CT1718 t1718 0 0.1f
M4643 t1715 nw603 t1718 0 nch w=1u l=180n
M4644 t1718 t1713 0 0 nch w=1u l=180n
M4645 nw605 t1714 vdd vdd pch w=2u l=180n
M4646 nw605 t1715 vdd vdd pch w=2u l=180n
CT1719 t1719 0 0.1f
M4647 nw605 t1714 t1719 0 nch w=1u l=180n
M4648 t1719 t1715 0 0 nch w=1u l=180n
Cnw605 nw605 0 2f
M4649 nw606 nw90 vdd vdd pch w=2u l=180n
M4650 nw606 nw533 vdd vdd pch w=2u l=180n
CT1720 t1720 0 0.1f
M4651 nw606 nw90 t1720 0 nch w=1u l=180n
M4652 t1720 nw533 0 0 nch w=1u l=180n
Cnw606 nw606 0 2f
M4653 nw607 nw604 vdd vdd pch w=2u l=180n
M4654 nw607 nw603 vdd vdd pch w=2u l=180n
CT1721 t1721 0 0.1f
M4655 nw607 nw604 t1721 0 nch w=1u l=180n
M4656 t1721 nw603 0 0 nch w=1u l=180n
Cnw607 nw607 0 2f
M4657 nw608 nw606 vdd vdd pch w=2u l=180n
M4658 nw608 nw607 vdd vdd pch w=2u l=180n
CT1722 t1722 0 0.1f
M4659 nw608 nw606 t1722 0 nch w=1u l=180n
M4660 t1722 nw607 0 0 nch w=1u l=180n
Cnw608 nw608 0 2f
CT1723 t1723 0 0.1f
CT1724 t1724 0 0.1f
CT1725 t1725 0 0.1f
M4661 t1723 nw91 vdd vdd pch w=2u l=180n
M4662 t1723 nw538 vdd vdd pch w=2u l=180n
CT1726 t1726 0 0.1f
M4663 t1723 nw91 t1726 0 nch w=1u l=180n
M4664 t1726 nw538 0 0 nch w=1u l=180n
M4665 t1724 nw91 vdd vdd pch w=2u l=180n
M4666 t1724 t1723 vdd vdd pch w=2u l=180n
CT1727 t1727 0 0.1f
M4667 t1724 nw91 t1727 0 nch w=1u l=180n
M4668 t1727 t1723 0 0 nch w=1u l=180n
M4669 t1725 nw538 vdd vdd pch w=2u l=180n
M4670 t1725 t1723 vdd vdd pch w=2u l=180n
CT1728 t1728 0 0.1f
M4671 t1725 nw538 t1728 0 nch w=1u l=180n
M4672 t1728 t1723 0 0 nch w=1u l=180n
M4673 nw609 t1724 vdd vdd pch w=2u l=180n
M4674 nw609 t1725 vdd vdd pch w=2u l=180n
CT1729 t1729 0 0.1f
M4675 nw609 t1724 t1729 0 nch w=1u l=180n
M4676 t1729 t1725 0 0 nch w=1u l=180n
Cnw609 nw609 0 2f
CT1730 t1730 0 0.1f
CT1731 t1731 0 0.1f
CT1732 t1732 0 0.1f
M4677 t1730 nw609 vdd vdd pch w=2u l=180n
M4678 t1730 nw608 vdd vdd pch w=2u l=180n
CT1733 t1733 0 0.1f
M4679 t1730 nw609 t1733 0 nch w=1u l=180n
M4680 t1733 nw608 0 0 nch w=1u l=180n
M4681 t1731 nw609 vdd vdd pch w=2u l=180n
M4682 t1731 t1730 vdd vdd pch w=2u l=180n
CT1734 t1734 0 0.1f
M4683 t1731 nw609 t1734 0 nch w=1u l=180n
M4684 t1734 t1730 0 0 nch w=1u l=180n
M4685 t1732 nw608 vdd vdd pch w=2u l=180n
M4686 t1732 t1730 vdd vdd pch w=2u l=180n
CT1735 t1735 0 0.1f
M4687 t1732 nw608 t1735 0 nch w=1u l=180n
M4688 t1735 t1730 0 0 nch w=1u l=180n
M4689 nw610 t1731 vdd vdd pch w=2u l=180n
M4690 nw610 t1732 vdd vdd pch w=2u l=180n
CT1736 t1736 0 0.1f
M4691 nw610 t1731 t1736 0 nch w=1u l=180n
M4692 t1736 t1732 0 0 nch w=1u l=180n
Cnw610 nw610 0 2f
M4693 nw611 nw91 vdd vdd pch w=2u l=180n
M4694 nw611 nw538 vdd vdd pch w=2u l=180n
CT1737 t1737 0 0.1f
M4695 nw611 nw91 t1737 0 nch w=1u l=180n
M4696 t1737 nw538 0 0 nch w=1u l=180n
Cnw611 nw611 0 2f
M4697 nw612 nw609 vdd vdd pch w=2u l=180n
M4698 nw612 nw608 vdd vdd pch w=2u l=180n
CT1738 t1738 0 0.1f
M4699 nw612 nw609 t1738 0 nch w=1u l=180n
M4700 t1738 nw608 0 0 nch w=1u l=180n
Cnw612 nw612 0 2f
M4701 nw613 nw611 vdd vdd pch w=2u l=180n
M4702 nw613 nw612 vdd vdd pch w=2u l=180n
CT1739 t1739 0 0.1f
M4703 nw613 nw611 t1739 0 nch w=1u l=180n
M4704 t1739 nw612 0 0 nch w=1u l=180n
Cnw613 nw613 0 2f
CT1740 t1740 0 0.1f
CT1741 t1741 0 0.1f
CT1742 t1742 0 0.1f
M4705 t1740 nw92 vdd vdd pch w=2u l=180n
M4706 t1740 nw543 vdd vdd pch w=2u l=180n
CT1743 t1743 0 0.1f
M4707 t1740 nw92 t1743 0 nch w=1u l=180n
M4708 t1743 nw543 0 0 nch w=1u l=180n
M4709 t1741 nw92 vdd vdd pch w=2u l=180n
M4710 t1741 t1740 vdd vdd pch w=2u l=180n
CT1744 t1744 0 0.1f
M4711 t1741 nw92 t1744 0 nch w=1u l=180n
M4712 t1744 t1740 0 0 nch w=1u l=180n
M4713 t1742 nw543 vdd vdd pch w=2u l=180n
M4714 t1742 t1740 vdd vdd pch w=2u l=180n
CT1745 t1745 0 0.1f
M4715 t1742 nw543 t1745 0 nch w=1u l=180n
M4716 t1745 t1740 0 0 nch w=1u l=180n
M4717 nw614 t1741 vdd vdd pch w=2u l=180n
M4718 nw614 t1742 vdd vdd pch w=2u l=180n
CT1746 t1746 0 0.1f
M4719 nw614 t1741 t1746 0 nch w=1u l=180n
M4720 t1746 t1742 0 0 nch w=1u l=180n
Cnw614 nw614 0 2f
CT1747 t1747 0 0.1f
CT1748 t1748 0 0.1f
CT1749 t1749 0 0.1f
M4721 t1747 nw614 vdd vdd pch w=2u l=180n
M4722 t1747 nw613 vdd vdd pch w=2u l=180n
CT1750 t1750 0 0.1f
M4723 t1747 nw614 t1750 0 nch w=1u l=180n
M4724 t1750 nw613 0 0 nch w=1u l=180n
M4725 t1748 nw614 vdd vdd pch w=2u l=180n
M4726 t1748 t1747 vdd vdd pch w=2u l=180n
CT1751 t1751 0 0.1f
M4727 t1748 nw614 t1751 0 nch w=1u l=180n
M4728 t1751 t1747 0 0 nch w=1u l=180n
M4729 t1749 nw613 vdd vdd pch w=2u l=180n
M4730 t1749 t1747 vdd vdd pch w=2u l=180n
CT1752 t1752 0 0.1f
M4731 t1749 nw613 t1752 0 nch w=1u l=180n
M4732 t1752 t1747 0 0 nch w=1u l=180n
M4733 nw615 t1748 vdd vdd pch w=2u l=180n
M4734 nw615 t1749 vdd vdd pch w=2u l=180n
CT1753 t1753 0 0.1f
M4735 nw615 t1748 t1753 0 nch w=1u l=180n
M4736 t1753 t1749 0 0 nch w=1u l=180n
Cnw615 nw615 0 2f
M4737 nw616 nw92 vdd vdd pch w=2u l=180n
M4738 nw616 nw543 vdd vdd pch w=2u l=180n
CT1754 t1754 0 0.1f
M4739 nw616 nw92 t1754 0 nch w=1u l=180n
M4740 t1754 nw543 0 0 nch w=1u l=180n
Cnw616 nw616 0 2f
M4741 nw617 nw614 vdd vdd pch w=2u l=180n
M4742 nw617 nw613 vdd vdd pch w=2u l=180n
CT1755 t1755 0 0.1f
M4743 nw617 nw614 t1755 0 nch w=1u l=180n
M4744 t1755 nw613 0 0 nch w=1u l=180n
Cnw617 nw617 0 2f
M4745 nw618 nw616 vdd vdd pch w=2u l=180n
M4746 nw618 nw617 vdd vdd pch w=2u l=180n
CT1756 t1756 0 0.1f
M4747 nw618 nw616 t1756 0 nch w=1u l=180n
M4748 t1756 nw617 0 0 nch w=1u l=180n
Cnw618 nw618 0 2f
CT1757 t1757 0 0.1f
CT1758 t1758 0 0.1f
CT1759 t1759 0 0.1f
M4749 t1757 nw93 vdd vdd pch w=2u l=180n
M4750 t1757 nw548 vdd vdd pch w=2u l=180n
CT1760 t1760 0 0.1f
M4751 t1757 nw93 t1760 0 nch w=1u l=180n
M4752 t1760 nw548 0 0 nch w=1u l=180n
M4753 t1758 nw93 vdd vdd pch w=2u l=180n
M4754 t1758 t1757 vdd vdd pch w=2u l=180n
CT1761 t1761 0 0.1f
M4755 t1758 nw93 t1761 0 nch w=1u l=180n
M4756 t1761 t1757 0 0 nch w=1u l=180n
M4757 t1759 nw548 vdd vdd pch w=2u l=180n
M4758 t1759 t1757 vdd vdd pch w=2u l=180n
CT1762 t1762 0 0.1f
M4759 t1759 nw548 t1762 0 nch w=1u l=180n
M4760 t1762 t1757 0 0 nch w=1u l=180n
M4761 nw619 t1758 vdd vdd pch w=2u l=180n
M4762 nw619 t1759 vdd vdd pch w=2u l=180n
CT1763 t1763 0 0.1f
M4763 nw619 t1758 t1763 0 nch w=1u l=180n
M4764 t1763 t1759 0 0 nch w=1u l=180n
Cnw619 nw619 0 2f
CT1764 t1764 0 0.1f
CT1765 t1765 0 0.1f
CT1766 t1766 0 0.1f
M4765 t1764 nw619 vdd vdd pch w=2u l=180n
M4766 t1764 nw618 vdd vdd pch w=2u l=180n
CT1767 t1767 0 0.1f
M4767 t1764 nw619 t1767 0 nch w=1u l=180n
M4768 t1767 nw618 0 0 nch w=1u l=180n
M4769 t1765 nw619 vdd vdd pch w=2u l=180n
M4770 t1765 t1764 vdd vdd pch w=2u l=180n
CT1768 t1768 0 0.1f
M4771 t1765 nw619 t1768 0 nch w=1u l=180n
M4772 t1768 t1764 0 0 nch w=1u l=180n
M4773 t1766 nw618 vdd vdd pch w=2u l=180n
M4774 t1766 t1764 vdd vdd pch w=2u l=180n
CT1769 t1769 0 0.1f
M4775 t1766 nw618 t1769 0 nch w=1u l=180n
M4776 t1769 t1764 0 0 nch w=1u l=180n
M4777 nw620 t1765 vdd vdd pch w=2u l=180n
M4778 nw620 t1766 vdd vdd pch w=2u l=180n
CT1770 t1770 0 0.1f
M4779 nw620 t1765 t1770 0 nch w=1u l=180n
M4780 t1770 t1766 0 0 nch w=1u l=180n
Cnw620 nw620 0 2f
M4781 nw621 nw93 vdd vdd pch w=2u l=180n
M4782 nw621 nw548 vdd vdd pch w=2u l=180n
CT1771 t1771 0 0.1f
M4783 nw621 nw93 t1771 0 nch w=1u l=180n
M4784 t1771 nw548 0 0 nch w=1u l=180n
Cnw621 nw621 0 2f
M4785 nw622 nw619 vdd vdd pch w=2u l=180n
M4786 nw622 nw618 vdd vdd pch w=2u l=180n
CT1772 t1772 0 0.1f
M4787 nw622 nw619 t1772 0 nch w=1u l=180n
M4788 t1772 nw618 0 0 nch w=1u l=180n
Cnw622 nw622 0 2f
M4789 nw623 nw621 vdd vdd pch w=2u l=180n
M4790 nw623 nw622 vdd vdd pch w=2u l=180n
CT1773 t1773 0 0.1f
M4791 nw623 nw621 t1773 0 nch w=1u l=180n
M4792 t1773 nw622 0 0 nch w=1u l=180n
Cnw623 nw623 0 2f
CT1774 t1774 0 0.1f
CT1775 t1775 0 0.1f
CT1776 t1776 0 0.1f
M4793 t1774 nw94 vdd vdd pch w=2u l=180n
M4794 t1774 nw553 vdd vdd pch w=2u l=180n
CT1777 t1777 0 0.1f
M4795 t1774 nw94 t1777 0 nch w=1u l=180n
M4796 t1777 nw553 0 0 nch w=1u l=180n
M4797 t1775 nw94 vdd vdd pch w=2u l=180n
M4798 t1775 t1774 vdd vdd pch w=2u l=180n
CT1778 t1778 0 0.1f
M4799 t1775 nw94 t1778 0 nch w=1u l=180n
M4800 t1778 t1774 0 0 nch w=1u l=180n
M4801 t1776 nw553 vdd vdd pch w=2u l=180n
M4802 t1776 t1774 vdd vdd pch w=2u l=180n
CT1779 t1779 0 0.1f
M4803 t1776 nw553 t1779 0 nch w=1u l=180n
M4804 t1779 t1774 0 0 nch w=1u l=180n
M4805 nw624 t1775 vdd vdd pch w=2u l=180n
M4806 nw624 t1776 vdd vdd pch w=2u l=180n
CT1780 t1780 0 0.1f
M4807 nw624 t1775 t1780 0 nch w=1u l=180n
M4808 t1780 t1776 0 0 nch w=1u l=180n
Cnw624 nw624 0 2f
CT1781 t1781 0 0.1f
CT1782 t1782 0 0.1f
CT1783 t1783 0 0.1f
M4809 t1781 nw624 vdd vdd pch w=2u l=180n
M4810 t1781 nw623 vdd vdd pch w=2u l=180n
CT1784 t1784 0 0.1f
M4811 t1781 nw624 t1784 0 nch w=1u l=180n
M4812 t1784 nw623 0 0 nch w=1u l=180n
M4813 t1782 nw624 vdd vdd pch w=2u l=180n
M4814 t1782 t1781 vdd vdd pch w=2u l=180n
CT1785 t1785 0 0.1f
M4815 t1782 nw624 t1785 0 nch w=1u l=180n
M4816 t1785 t1781 0 0 nch w=1u l=180n
M4817 t1783 nw623 vdd vdd pch w=2u l=180n
M4818 t1783 t1781 vdd vdd pch w=2u l=180n
CT1786 t1786 0 0.1f
M4819 t1783 nw623 t1786 0 nch w=1u l=180n
M4820 t1786 t1781 0 0 nch w=1u l=180n
M4821 nw625 t1782 vdd vdd pch w=2u l=180n
M4822 nw625 t1783 vdd vdd pch w=2u l=180n
CT1787 t1787 0 0.1f
M4823 nw625 t1782 t1787 0 nch w=1u l=180n
M4824 t1787 t1783 0 0 nch w=1u l=180n
Cnw625 nw625 0 2f
M4825 nw626 nw94 vdd vdd pch w=2u l=180n
M4826 nw626 nw553 vdd vdd pch w=2u l=180n
CT1788 t1788 0 0.1f
M4827 nw626 nw94 t1788 0 nch w=1u l=180n
M4828 t1788 nw553 0 0 nch w=1u l=180n
Cnw626 nw626 0 2f
M4829 nw627 nw624 vdd vdd pch w=2u l=180n
M4830 nw627 nw623 vdd vdd pch w=2u l=180n
CT1789 t1789 0 0.1f
M4831 nw627 nw624 t1789 0 nch w=1u l=180n
M4832 t1789 nw623 0 0 nch w=1u l=180n
Cnw627 nw627 0 2f
M4833 nw628 nw626 vdd vdd pch w=2u l=180n
M4834 nw628 nw627 vdd vdd pch w=2u l=180n
CT1790 t1790 0 0.1f
M4835 nw628 nw626 t1790 0 nch w=1u l=180n
M4836 t1790 nw627 0 0 nch w=1u l=180n
Cnw628 nw628 0 2f
CT1791 t1791 0 0.1f
CT1792 t1792 0 0.1f
CT1793 t1793 0 0.1f
M4837 t1791 nw95 vdd vdd pch w=2u l=180n
M4838 t1791 nw558 vdd vdd pch w=2u l=180n
CT1794 t1794 0 0.1f
M4839 t1791 nw95 t1794 0 nch w=1u l=180n
M4840 t1794 nw558 0 0 nch w=1u l=180n
M4841 t1792 nw95 vdd vdd pch w=2u l=180n
M4842 t1792 t1791 vdd vdd pch w=2u l=180n
CT1795 t1795 0 0.1f
M4843 t1792 nw95 t1795 0 nch w=1u l=180n
M4844 t1795 t1791 0 0 nch w=1u l=180n
M4845 t1793 nw558 vdd vdd pch w=2u l=180n
M4846 t1793 t1791 vdd vdd pch w=2u l=180n
CT1796 t1796 0 0.1f
M4847 t1793 nw558 t1796 0 nch w=1u l=180n
M4848 t1796 t1791 0 0 nch w=1u l=180n
M4849 nw629 t1792 vdd vdd pch w=2u l=180n
M4850 nw629 t1793 vdd vdd pch w=2u l=180n
CT1797 t1797 0 0.1f
M4851 nw629 t1792 t1797 0 nch w=1u l=180n
M4852 t1797 t1793 0 0 nch w=1u l=180n
Cnw629 nw629 0 2f
CT1798 t1798 0 0.1f
CT1799 t1799 0 0.1f
CT1800 t1800 0 0.1f
M4853 t1798 nw629 vdd vdd pch w=2u l=180n
M4854 t1798 nw628 vdd vdd pch w=2u l=180n
CT1801 t1801 0 0.1f
M4855 t1798 nw629 t1801 0 nch w=1u l=180n
M4856 t1801 nw628 0 0 nch w=1u l=180n
M4857 t1799 nw629 vdd vdd pch w=2u l=180n
M4858 t1799 t1798 vdd vdd pch w=2u l=180n
CT1802 t1802 0 0.1f
M4859 t1799 nw629 t1802 0 nch w=1u l=180n
M4860 t1802 t1798 0 0 nch w=1u l=180n
M4861 t1800 nw628 vdd vdd pch w=2u l=180n
M4862 t1800 t1798 vdd vdd pch w=2u l=180n
CT1803 t1803 0 0.1f
M4863 t1800 nw628 t1803 0 nch w=1u l=180n
M4864 t1803 t1798 0 0 nch w=1u l=180n
M4865 nw630 t1799 vdd vdd pch w=2u l=180n
M4866 nw630 t1800 vdd vdd pch w=2u l=180n
CT1804 t1804 0 0.1f
M4867 nw630 t1799 t1804 0 nch w=1u l=180n
M4868 t1804 t1800 0 0 nch w=1u l=180n
Cnw630 nw630 0 2f
M4869 nw631 nw95 vdd vdd pch w=2u l=180n
M4870 nw631 nw558 vdd vdd pch w=2u l=180n
CT1805 t1805 0 0.1f
M4871 nw631 nw95 t1805 0 nch w=1u l=180n
M4872 t1805 nw558 0 0 nch w=1u l=180n
Cnw631 nw631 0 2f
M4873 nw632 nw629 vdd vdd pch w=2u l=180n
M4874 nw632 nw628 vdd vdd pch w=2u l=180n
CT1806 t1806 0 0.1f
M4875 nw632 nw629 t1806 0 nch w=1u l=180n
M4876 t1806 nw628 0 0 nch w=1u l=180n
Cnw632 nw632 0 2f
M4877 nw633 nw631 vdd vdd pch w=2u l=180n
M4878 nw633 nw632 vdd vdd pch w=2u l=180n
CT1807 t1807 0 0.1f
M4879 nw633 nw631 t1807 0 nch w=1u l=180n
M4880 t1807 nw632 0 0 nch w=1u l=180n
Cnw633 nw633 0 2f
CT1808 t1808 0 0.1f
CT1809 t1809 0 0.1f
CT1810 t1810 0 0.1f
M4881 t1808 nw96 vdd vdd pch w=2u l=180n
M4882 t1808 nw561 vdd vdd pch w=2u l=180n
CT1811 t1811 0 0.1f
M4883 t1808 nw96 t1811 0 nch w=1u l=180n
M4884 t1811 nw561 0 0 nch w=1u l=180n
M4885 t1809 nw96 vdd vdd pch w=2u l=180n
M4886 t1809 t1808 vdd vdd pch w=2u l=180n
CT1812 t1812 0 0.1f
M4887 t1809 nw96 t1812 0 nch w=1u l=180n
M4888 t1812 t1808 0 0 nch w=1u l=180n
M4889 t1810 nw561 vdd vdd pch w=2u l=180n
M4890 t1810 t1808 vdd vdd pch w=2u l=180n
CT1813 t1813 0 0.1f
M4891 t1810 nw561 t1813 0 nch w=1u l=180n
M4892 t1813 t1808 0 0 nch w=1u l=180n
M4893 nw634 t1809 vdd vdd pch w=2u l=180n
M4894 nw634 t1810 vdd vdd pch w=2u l=180n
CT1814 t1814 0 0.1f
M4895 nw634 t1809 t1814 0 nch w=1u l=180n
M4896 t1814 t1810 0 0 nch w=1u l=180n
Cnw634 nw634 0 2f
CT1815 t1815 0 0.1f
CT1816 t1816 0 0.1f
CT1817 t1817 0 0.1f
M4897 t1815 nw634 vdd vdd pch w=2u l=180n
M4898 t1815 nw633 vdd vdd pch w=2u l=180n
CT1818 t1818 0 0.1f
M4899 t1815 nw634 t1818 0 nch w=1u l=180n
M4900 t1818 nw633 0 0 nch w=1u l=180n
M4901 t1816 nw634 vdd vdd pch w=2u l=180n
M4902 t1816 t1815 vdd vdd pch w=2u l=180n
CT1819 t1819 0 0.1f
M4903 t1816 nw634 t1819 0 nch w=1u l=180n
M4904 t1819 t1815 0 0 nch w=1u l=180n
M4905 t1817 nw633 vdd vdd pch w=2u l=180n
M4906 t1817 t1815 vdd vdd pch w=2u l=180n
CT1820 t1820 0 0.1f
M4907 t1817 nw633 t1820 0 nch w=1u l=180n
M4908 t1820 t1815 0 0 nch w=1u l=180n
M4909 nw635 t1816 vdd vdd pch w=2u l=180n
M4910 nw635 t1817 vdd vdd pch w=2u l=180n
CT1821 t1821 0 0.1f
M4911 nw635 t1816 t1821 0 nch w=1u l=180n
M4912 t1821 t1817 0 0 nch w=1u l=180n
Cnw635 nw635 0 2f
M4913 nw636 nw96 vdd vdd pch w=2u l=180n
M4914 nw636 nw561 vdd vdd pch w=2u l=180n
CT1822 t1822 0 0.1f
M4915 nw636 nw96 t1822 0 nch w=1u l=180n
M4916 t1822 nw561 0 0 nch w=1u l=180n
Cnw636 nw636 0 2f
M4917 nw637 nw634 vdd vdd pch w=2u l=180n
M4918 nw637 nw633 vdd vdd pch w=2u l=180n
CT1823 t1823 0 0.1f
M4919 nw637 nw634 t1823 0 nch w=1u l=180n
M4920 t1823 nw633 0 0 nch w=1u l=180n
Cnw637 nw637 0 2f
M4921 nw638 nw636 vdd vdd pch w=2u l=180n
M4922 nw638 nw637 vdd vdd pch w=2u l=180n
CT1824 t1824 0 0.1f
M4923 nw638 nw636 t1824 0 nch w=1u l=180n
M4924 t1824 nw637 0 0 nch w=1u l=180n
Cnw638 nw638 0 2f
CT1825 t1825 0 0.1f
CT1826 t1826 0 0.1f
CT1827 t1827 0 0.1f
M4925 t1825 nw97 vdd vdd pch w=2u l=180n
M4926 t1825 nw565 vdd vdd pch w=2u l=180n
CT1828 t1828 0 0.1f
M4927 t1825 nw97 t1828 0 nch w=1u l=180n
M4928 t1828 nw565 0 0 nch w=1u l=180n
M4929 t1826 nw97 vdd vdd pch w=2u l=180n
M4930 t1826 t1825 vdd vdd pch w=2u l=180n
CT1829 t1829 0 0.1f
M4931 t1826 nw97 t1829 0 nch w=1u l=180n
M4932 t1829 t1825 0 0 nch w=1u l=180n
M4933 t1827 nw565 vdd vdd pch w=2u l=180n
M4934 t1827 t1825 vdd vdd pch w=2u l=180n
CT1830 t1830 0 0.1f
M4935 t1827 nw565 t1830 0 nch w=1u l=180n
M4936 t1830 t1825 0 0 nch w=1u l=180n
M4937 nw639 t1826 vdd vdd pch w=2u l=180n
M4938 nw639 t1827 vdd vdd pch w=2u l=180n
CT1831 t1831 0 0.1f
M4939 nw639 t1826 t1831 0 nch w=1u l=180n
M4940 t1831 t1827 0 0 nch w=1u l=180n
Cnw639 nw639 0 2f
CT1832 t1832 0 0.1f
M4941 t1832 nw97 vdd vdd pch w=2u l=180n
M4942 t1832 nw565 vdd vdd pch w=2u l=180n
CT1833 t1833 0 0.1f
M4943 t1832 nw97 t1833 0 nch w=1u l=180n
M4944 t1833 nw565 0 0 nch w=1u l=180n
M4945 nw640 t1832 vdd vdd pch w=2u l=180n
M4946 nw640 t1832 0 0 nch w=1u l=180n
Cnw640 nw640 0 2f
CT1834 t1834 0 0.1f
CT1835 t1835 0 0.1f
CT1836 t1836 0 0.1f
M4947 t1834 nw98 vdd vdd pch w=2u l=180n
M4948 t1834 nw570 vdd vdd pch w=2u l=180n
CT1837 t1837 0 0.1f
M4949 t1834 nw98 t1837 0 nch w=1u l=180n
M4950 t1837 nw570 0 0 nch w=1u l=180n
M4951 t1835 nw98 vdd vdd pch w=2u l=180n
M4952 t1835 t1834 vdd vdd pch w=2u l=180n
CT1838 t1838 0 0.1f
M4953 t1835 nw98 t1838 0 nch w=1u l=180n
M4954 t1838 t1834 0 0 nch w=1u l=180n
M4955 t1836 nw570 vdd vdd pch w=2u l=180n
M4956 t1836 t1834 vdd vdd pch w=2u l=180n
CT1839 t1839 0 0.1f
M4957 t1836 nw570 t1839 0 nch w=1u l=180n
M4958 t1839 t1834 0 0 nch w=1u l=180n
M4959 nw641 t1835 vdd vdd pch w=2u l=180n
M4960 nw641 t1836 vdd vdd pch w=2u l=180n
CT1840 t1840 0 0.1f
M4961 nw641 t1835 t1840 0 nch w=1u l=180n
M4962 t1840 t1836 0 0 nch w=1u l=180n
Cnw641 nw641 0 2f
CT1841 t1841 0 0.1f
CT1842 t1842 0 0.1f
CT1843 t1843 0 0.1f
M4963 t1841 nw641 vdd vdd pch w=2u l=180n
M4964 t1841 nw640 vdd vdd pch w=2u l=180n
CT1844 t1844 0 0.1f
M4965 t1841 nw641 t1844 0 nch w=1u l=180n
M4966 t1844 nw640 0 0 nch w=1u l=180n
M4967 t1842 nw641 vdd vdd pch w=2u l=180n
M4968 t1842 t1841 vdd vdd pch w=2u l=180n
CT1845 t1845 0 0.1f
M4969 t1842 nw641 t1845 0 nch w=1u l=180n
M4970 t1845 t1841 0 0 nch w=1u l=180n
M4971 t1843 nw640 vdd vdd pch w=2u l=180n
M4972 t1843 t1841 vdd vdd pch w=2u l=180n
CT1846 t1846 0 0.1f
M4973 t1843 nw640 t1846 0 nch w=1u l=180n
M4974 t1846 t1841 0 0 nch w=1u l=180n
M4975 nw642 t1842 vdd vdd pch w=2u l=180n
M4976 nw642 t1843 vdd vdd pch w=2u l=180n
CT1847 t1847 0 0.1f
M4977 nw642 t1842 t1847 0 nch w=1u l=180n
M4978 t1847 t1843 0 0 nch w=1u l=180n
Cnw642 nw642 0 2f
M4979 nw643 nw98 vdd vdd pch w=2u l=180n
M4980 nw643 nw570 vdd vdd pch w=2u l=180n
CT1848 t1848 0 0.1f
M4981 nw643 nw98 t1848 0 nch w=1u l=180n
M4982 t1848 nw570 0 0 nch w=1u l=180n
Cnw643 nw643 0 2f
M4983 nw644 nw641 vdd vdd pch w=2u l=180n
M4984 nw644 nw640 vdd vdd pch w=2u l=180n
CT1849 t1849 0 0.1f
M4985 nw644 nw641 t1849 0 nch w=1u l=180n
M4986 t1849 nw640 0 0 nch w=1u l=180n
Cnw644 nw644 0 2f
M4987 nw645 nw643 vdd vdd pch w=2u l=180n
M4988 nw645 nw644 vdd vdd pch w=2u l=180n
CT1850 t1850 0 0.1f
M4989 nw645 nw643 t1850 0 nch w=1u l=180n
M4990 t1850 nw644 0 0 nch w=1u l=180n
Cnw645 nw645 0 2f
CT1851 t1851 0 0.1f
CT1852 t1852 0 0.1f
CT1853 t1853 0 0.1f
M4991 t1851 nw99 vdd vdd pch w=2u l=180n
M4992 t1851 nw575 vdd vdd pch w=2u l=180n
CT1854 t1854 0 0.1f
M4993 t1851 nw99 t1854 0 nch w=1u l=180n
M4994 t1854 nw575 0 0 nch w=1u l=180n
M4995 t1852 nw99 vdd vdd pch w=2u l=180n
M4996 t1852 t1851 vdd vdd pch w=2u l=180n
CT1855 t1855 0 0.1f
M4997 t1852 nw99 t1855 0 nch w=1u l=180n
M4998 t1855 t1851 0 0 nch w=1u l=180n
M4999 t1853 nw575 vdd vdd pch w=2u l=180n
M5000 t1853 t1851 vdd vdd pch w=2u l=180n
CT1856 t1856 0 0.1f
M5001 t1853 nw575 t1856 0 nch w=1u l=180n
M5002 t1856 t1851 0 0 nch w=1u l=180n
M5003 nw646 t1852 vdd vdd pch w=2u l=180n
M5004 nw646 t1853 vdd vdd pch w=2u l=180n
CT1857 t1857 0 0.1f
M5005 nw646 t1852 t1857 0 nch w=1u l=180n
M5006 t1857 t1853 0 0 nch w=1u l=180n
Cnw646 nw646 0 2f
CT1858 t1858 0 0.1f
CT1859 t1859 0 0.1f
CT1860 t1860 0 0.1f
M5007 t1858 nw646 vdd vdd pch w=2u l=180n
M5008 t1858 nw645 vdd vdd pch w=2u l=180n
CT1861 t1861 0 0.1f
M5009 t1858 nw646 t1861 0 nch w=1u l=180n
M5010 t1861 nw645 0 0 nch w=1u l=180n
M5011 t1859 nw646 vdd vdd pch w=2u l=180n
M5012 t1859 t1858 vdd vdd pch w=2u l=180n
CT1862 t1862 0 0.1f
M5013 t1859 nw646 t1862 0 nch w=1u l=180n
M5014 t1862 t1858 0 0 nch w=1u l=180n
M5015 t1860 nw645 vdd vdd pch w=2u l=180n
M5016 t1860 t1858 vdd vdd pch w=2u l=180n
CT1863 t1863 0 0.1f
M5017 t1860 nw645 t1863 0 nch w=1u l=180n
M5018 t1863 t1858 0 0 nch w=1u l=180n
M5019 nw647 t1859 vdd vdd pch w=2u l=180n
M5020 nw647 t1860 vdd vdd pch w=2u l=180n
CT1864 t1864 0 0.1f
M5021 nw647 t1859 t1864 0 nch w=1u l=180n
M5022 t1864 t1860 0 0 nch w=1u l=180n
Cnw647 nw647 0 2f
M5023 nw648 nw99 vdd vdd pch w=2u l=180n
M5024 nw648 nw575 vdd vdd pch w=2u l=180n
CT1865 t1865 0 0.1f
M5025 nw648 nw99 t1865 0 nch w=1u l=180n
M5026 t1865 nw575 0 0 nch w=1u l=180n
Cnw648 nw648 0 2f
M5027 nw649 nw646 vdd vdd pch w=2u l=180n
M5028 nw649 nw645 vdd vdd pch w=2u l=180n
CT1866 t1866 0 0.1f
M5029 nw649 nw646 t1866 0 nch w=1u l=180n
M5030 t1866 nw645 0 0 nch w=1u l=180n
Cnw649 nw649 0 2f
M5031 nw650 nw648 vdd vdd pch w=2u l=180n
M5032 nw650 nw649 vdd vdd pch w=2u l=180n
CT1867 t1867 0 0.1f
M5033 nw650 nw648 t1867 0 nch w=1u l=180n
M5034 t1867 nw649 0 0 nch w=1u l=180n
Cnw650 nw650 0 2f
CT1868 t1868 0 0.1f
CT1869 t1869 0 0.1f
CT1870 t1870 0 0.1f
M5035 t1868 nw100 vdd vdd pch w=2u l=180n
M5036 t1868 nw580 vdd vdd pch w=2u l=180n
CT1871 t1871 0 0.1f
M5037 t1868 nw100 t1871 0 nch w=1u l=180n
M5038 t1871 nw580 0 0 nch w=1u l=180n
M5039 t1869 nw100 vdd vdd pch w=2u l=180n
M5040 t1869 t1868 vdd vdd pch w=2u l=180n
CT1872 t1872 0 0.1f
M5041 t1869 nw100 t1872 0 nch w=1u l=180n
M5042 t1872 t1868 0 0 nch w=1u l=180n
M5043 t1870 nw580 vdd vdd pch w=2u l=180n
M5044 t1870 t1868 vdd vdd pch w=2u l=180n
CT1873 t1873 0 0.1f
M5045 t1870 nw580 t1873 0 nch w=1u l=180n
M5046 t1873 t1868 0 0 nch w=1u l=180n
M5047 nw651 t1869 vdd vdd pch w=2u l=180n
M5048 nw651 t1870 vdd vdd pch w=2u l=180n
CT1874 t1874 0 0.1f
M5049 nw651 t1869 t1874 0 nch w=1u l=180n
M5050 t1874 t1870 0 0 nch w=1u l=180n
Cnw651 nw651 0 2f
CT1875 t1875 0 0.1f
CT1876 t1876 0 0.1f
CT1877 t1877 0 0.1f
M5051 t1875 nw651 vdd vdd pch w=2u l=180n
M5052 t1875 nw650 vdd vdd pch w=2u l=180n
CT1878 t1878 0 0.1f
M5053 t1875 nw651 t1878 0 nch w=1u l=180n
M5054 t1878 nw650 0 0 nch w=1u l=180n
M5055 t1876 nw651 vdd vdd pch w=2u l=180n
M5056 t1876 t1875 vdd vdd pch w=2u l=180n
CT1879 t1879 0 0.1f
M5057 t1876 nw651 t1879 0 nch w=1u l=180n
M5058 t1879 t1875 0 0 nch w=1u l=180n
M5059 t1877 nw650 vdd vdd pch w=2u l=180n
M5060 t1877 t1875 vdd vdd pch w=2u l=180n
CT1880 t1880 0 0.1f
M5061 t1877 nw650 t1880 0 nch w=1u l=180n
M5062 t1880 t1875 0 0 nch w=1u l=180n
M5063 nw652 t1876 vdd vdd pch w=2u l=180n
M5064 nw652 t1877 vdd vdd pch w=2u l=180n
CT1881 t1881 0 0.1f
M5065 nw652 t1876 t1881 0 nch w=1u l=180n
M5066 t1881 t1877 0 0 nch w=1u l=180n
Cnw652 nw652 0 2f
M5067 nw653 nw100 vdd vdd pch w=2u l=180n
M5068 nw653 nw580 vdd vdd pch w=2u l=180n
CT1882 t1882 0 0.1f
M5069 nw653 nw100 t1882 0 nch w=1u l=180n
M5070 t1882 nw580 0 0 nch w=1u l=180n
Cnw653 nw653 0 2f
M5071 nw654 nw651 vdd vdd pch w=2u l=180n
M5072 nw654 nw650 vdd vdd pch w=2u l=180n
CT1883 t1883 0 0.1f
M5073 nw654 nw651 t1883 0 nch w=1u l=180n
M5074 t1883 nw650 0 0 nch w=1u l=180n
Cnw654 nw654 0 2f
M5075 nw655 nw653 vdd vdd pch w=2u l=180n
M5076 nw655 nw654 vdd vdd pch w=2u l=180n
CT1884 t1884 0 0.1f
M5077 nw655 nw653 t1884 0 nch w=1u l=180n
M5078 t1884 nw654 0 0 nch w=1u l=180n
Cnw655 nw655 0 2f
CT1885 t1885 0 0.1f
CT1886 t1886 0 0.1f
CT1887 t1887 0 0.1f
M5079 t1885 nw101 vdd vdd pch w=2u l=180n
M5080 t1885 nw585 vdd vdd pch w=2u l=180n
CT1888 t1888 0 0.1f
M5081 t1885 nw101 t1888 0 nch w=1u l=180n
M5082 t1888 nw585 0 0 nch w=1u l=180n
M5083 t1886 nw101 vdd vdd pch w=2u l=180n
M5084 t1886 t1885 vdd vdd pch w=2u l=180n
CT1889 t1889 0 0.1f
M5085 t1886 nw101 t1889 0 nch w=1u l=180n
M5086 t1889 t1885 0 0 nch w=1u l=180n
M5087 t1887 nw585 vdd vdd pch w=2u l=180n
M5088 t1887 t1885 vdd vdd pch w=2u l=180n
CT1890 t1890 0 0.1f
M5089 t1887 nw585 t1890 0 nch w=1u l=180n
M5090 t1890 t1885 0 0 nch w=1u l=180n
M5091 nw656 t1886 vdd vdd pch w=2u l=180n
M5092 nw656 t1887 vdd vdd pch w=2u l=180n
CT1891 t1891 0 0.1f
M5093 nw656 t1886 t1891 0 nch w=1u l=180n
M5094 t1891 t1887 0 0 nch w=1u l=180n
Cnw656 nw656 0 2f
CT1892 t1892 0 0.1f
CT1893 t1893 0 0.1f
CT1894 t1894 0 0.1f
M5095 t1892 nw656 vdd vdd pch w=2u l=180n
M5096 t1892 nw655 vdd vdd pch w=2u l=180n
CT1895 t1895 0 0.1f
M5097 t1892 nw656 t1895 0 nch w=1u l=180n
M5098 t1895 nw655 0 0 nch w=1u l=180n
M5099 t1893 nw656 vdd vdd pch w=2u l=180n
M5100 t1893 t1892 vdd vdd pch w=2u l=180n
CT1896 t1896 0 0.1f
M5101 t1893 nw656 t1896 0 nch w=1u l=180n
M5102 t1896 t1892 0 0 nch w=1u l=180n
M5103 t1894 nw655 vdd vdd pch w=2u l=180n
M5104 t1894 t1892 vdd vdd pch w=2u l=180n
CT1897 t1897 0 0.1f
M5105 t1894 nw655 t1897 0 nch w=1u l=180n
M5106 t1897 t1892 0 0 nch w=1u l=180n
M5107 nw657 t1893 vdd vdd pch w=2u l=180n
M5108 nw657 t1894 vdd vdd pch w=2u l=180n
CT1898 t1898 0 0.1f
M5109 nw657 t1893 t1898 0 nch w=1u l=180n
M5110 t1898 t1894 0 0 nch w=1u l=180n
Cnw657 nw657 0 2f
M5111 nw658 nw101 vdd vdd pch w=2u l=180n
M5112 nw658 nw585 vdd vdd pch w=2u l=180n
CT1899 t1899 0 0.1f
M5113 nw658 nw101 t1899 0 nch w=1u l=180n
M5114 t1899 nw585 0 0 nch w=1u l=180n
Cnw658 nw658 0 2f
M5115 nw659 nw656 vdd vdd pch w=2u l=180n
M5116 nw659 nw655 vdd vdd pch w=2u l=180n
CT1900 t1900 0 0.1f
M5117 nw659 nw656 t1900 0 nch w=1u l=180n
M5118 t1900 nw655 0 0 nch w=1u l=180n
Cnw659 nw659 0 2f
M5119 nw660 nw658 vdd vdd pch w=2u l=180n
M5120 nw660 nw659 vdd vdd pch w=2u l=180n
CT1901 t1901 0 0.1f
M5121 nw660 nw658 t1901 0 nch w=1u l=180n
M5122 t1901 nw659 0 0 nch w=1u l=180n
Cnw660 nw660 0 2f
CT1902 t1902 0 0.1f
CT1903 t1903 0 0.1f
CT1904 t1904 0 0.1f
M5123 t1902 nw102 vdd vdd pch w=2u l=180n
M5124 t1902 nw590 vdd vdd pch w=2u l=180n
CT1905 t1905 0 0.1f
M5125 t1902 nw102 t1905 0 nch w=1u l=180n
M5126 t1905 nw590 0 0 nch w=1u l=180n
M5127 t1903 nw102 vdd vdd pch w=2u l=180n
M5128 t1903 t1902 vdd vdd pch w=2u l=180n
CT1906 t1906 0 0.1f
M5129 t1903 nw102 t1906 0 nch w=1u l=180n
M5130 t1906 t1902 0 0 nch w=1u l=180n
M5131 t1904 nw590 vdd vdd pch w=2u l=180n
M5132 t1904 t1902 vdd vdd pch w=2u l=180n
CT1907 t1907 0 0.1f
M5133 t1904 nw590 t1907 0 nch w=1u l=180n
M5134 t1907 t1902 0 0 nch w=1u l=180n
M5135 nw661 t1903 vdd vdd pch w=2u l=180n
M5136 nw661 t1904 vdd vdd pch w=2u l=180n
CT1908 t1908 0 0.1f
M5137 nw661 t1903 t1908 0 nch w=1u l=180n
M5138 t1908 t1904 0 0 nch w=1u l=180n
Cnw661 nw661 0 2f
CT1909 t1909 0 0.1f
CT1910 t1910 0 0.1f
CT1911 t1911 0 0.1f
M5139 t1909 nw661 vdd vdd pch w=2u l=180n
M5140 t1909 nw660 vdd vdd pch w=2u l=180n
CT1912 t1912 0 0.1f
M5141 t1909 nw661 t1912 0 nch w=1u l=180n
M5142 t1912 nw660 0 0 nch w=1u l=180n
M5143 t1910 nw661 vdd vdd pch w=2u l=180n
M5144 t1910 t1909 vdd vdd pch w=2u l=180n
CT1913 t1913 0 0.1f
M5145 t1910 nw661 t1913 0 nch w=1u l=180n
M5146 t1913 t1909 0 0 nch w=1u l=180n
M5147 t1911 nw660 vdd vdd pch w=2u l=180n
M5148 t1911 t1909 vdd vdd pch w=2u l=180n
CT1914 t1914 0 0.1f
M5149 t1911 nw660 t1914 0 nch w=1u l=180n
M5150 t1914 t1909 0 0 nch w=1u l=180n
M5151 nw662 t1910 vdd vdd pch w=2u l=180n
M5152 nw662 t1911 vdd vdd pch w=2u l=180n
CT1915 t1915 0 0.1f
M5153 nw662 t1910 t1915 0 nch w=1u l=180n
M5154 t1915 t1911 0 0 nch w=1u l=180n
Cnw662 nw662 0 2f
M5155 nw663 nw102 vdd vdd pch w=2u l=180n
M5156 nw663 nw590 vdd vdd pch w=2u l=180n
CT1916 t1916 0 0.1f
M5157 nw663 nw102 t1916 0 nch w=1u l=180n
M5158 t1916 nw590 0 0 nch w=1u l=180n
Cnw663 nw663 0 2f
M5159 nw664 nw661 vdd vdd pch w=2u l=180n
M5160 nw664 nw660 vdd vdd pch w=2u l=180n
CT1917 t1917 0 0.1f
M5161 nw664 nw661 t1917 0 nch w=1u l=180n
M5162 t1917 nw660 0 0 nch w=1u l=180n
Cnw664 nw664 0 2f
M5163 nw665 nw663 vdd vdd pch w=2u l=180n
M5164 nw665 nw664 vdd vdd pch w=2u l=180n
CT1918 t1918 0 0.1f
M5165 nw665 nw663 t1918 0 nch w=1u l=180n
M5166 t1918 nw664 0 0 nch w=1u l=180n
Cnw665 nw665 0 2f
CT1919 t1919 0 0.1f
CT1920 t1920 0 0.1f
CT1921 t1921 0 0.1f
M5167 t1919 nw103 vdd vdd pch w=2u l=180n
M5168 t1919 nw595 vdd vdd pch w=2u l=180n
CT1922 t1922 0 0.1f
M5169 t1919 nw103 t1922 0 nch w=1u l=180n
M5170 t1922 nw595 0 0 nch w=1u l=180n
M5171 t1920 nw103 vdd vdd pch w=2u l=180n
M5172 t1920 t1919 vdd vdd pch w=2u l=180n
CT1923 t1923 0 0.1f
M5173 t1920 nw103 t1923 0 nch w=1u l=180n
M5174 t1923 t1919 0 0 nch w=1u l=180n
M5175 t1921 nw595 vdd vdd pch w=2u l=180n
M5176 t1921 t1919 vdd vdd pch w=2u l=180n
CT1924 t1924 0 0.1f
M5177 t1921 nw595 t1924 0 nch w=1u l=180n
M5178 t1924 t1919 0 0 nch w=1u l=180n
M5179 nw666 t1920 vdd vdd pch w=2u l=180n
M5180 nw666 t1921 vdd vdd pch w=2u l=180n
CT1925 t1925 0 0.1f
M5181 nw666 t1920 t1925 0 nch w=1u l=180n
M5182 t1925 t1921 0 0 nch w=1u l=180n
Cnw666 nw666 0 2f
CT1926 t1926 0 0.1f
CT1927 t1927 0 0.1f
CT1928 t1928 0 0.1f
M5183 t1926 nw666 vdd vdd pch w=2u l=180n
M5184 t1926 nw665 vdd vdd pch w=2u l=180n
CT1929 t1929 0 0.1f
M5185 t1926 nw666 t1929 0 nch w=1u l=180n
M5186 t1929 nw665 0 0 nch w=1u l=180n
M5187 t1927 nw666 vdd vdd pch w=2u l=180n
M5188 t1927 t1926 vdd vdd pch w=2u l=180n
CT1930 t1930 0 0.1f
M5189 t1927 nw666 t1930 0 nch w=1u l=180n
M5190 t1930 t1926 0 0 nch w=1u l=180n
M5191 t1928 nw665 vdd vdd pch w=2u l=180n
M5192 t1928 t1926 vdd vdd pch w=2u l=180n
CT1931 t1931 0 0.1f
M5193 t1928 nw665 t1931 0 nch w=1u l=180n
M5194 t1931 t1926 0 0 nch w=1u l=180n
M5195 nw667 t1927 vdd vdd pch w=2u l=180n
M5196 nw667 t1928 vdd vdd pch w=2u l=180n
CT1932 t1932 0 0.1f
M5197 nw667 t1927 t1932 0 nch w=1u l=180n
M5198 t1932 t1928 0 0 nch w=1u l=180n
Cnw667 nw667 0 2f
M5199 nw668 nw103 vdd vdd pch w=2u l=180n
M5200 nw668 nw595 vdd vdd pch w=2u l=180n
CT1933 t1933 0 0.1f
M5201 nw668 nw103 t1933 0 nch w=1u l=180n
M5202 t1933 nw595 0 0 nch w=1u l=180n
Cnw668 nw668 0 2f
M5203 nw669 nw666 vdd vdd pch w=2u l=180n
M5204 nw669 nw665 vdd vdd pch w=2u l=180n
CT1934 t1934 0 0.1f
M5205 nw669 nw666 t1934 0 nch w=1u l=180n
M5206 t1934 nw665 0 0 nch w=1u l=180n
Cnw669 nw669 0 2f
M5207 nw670 nw668 vdd vdd pch w=2u l=180n
M5208 nw670 nw669 vdd vdd pch w=2u l=180n
CT1935 t1935 0 0.1f
M5209 nw670 nw668 t1935 0 nch w=1u l=180n
M5210 t1935 nw669 0 0 nch w=1u l=180n
Cnw670 nw670 0 2f
CT1936 t1936 0 0.1f
CT1937 t1937 0 0.1f
CT1938 t1938 0 0.1f
M5211 t1936 nw104 vdd vdd pch w=2u l=180n
M5212 t1936 nw600 vdd vdd pch w=2u l=180n
CT1939 t1939 0 0.1f
M5213 t1936 nw104 t1939 0 nch w=1u l=180n
M5214 t1939 nw600 0 0 nch w=1u l=180n
M5215 t1937 nw104 vdd vdd pch w=2u l=180n
M5216 t1937 t1936 vdd vdd pch w=2u l=180n
CT1940 t1940 0 0.1f
M5217 t1937 nw104 t1940 0 nch w=1u l=180n
M5218 t1940 t1936 0 0 nch w=1u l=180n
M5219 t1938 nw600 vdd vdd pch w=2u l=180n
M5220 t1938 t1936 vdd vdd pch w=2u l=180n
CT1941 t1941 0 0.1f
M5221 t1938 nw600 t1941 0 nch w=1u l=180n
M5222 t1941 t1936 0 0 nch w=1u l=180n
M5223 nw671 t1937 vdd vdd pch w=2u l=180n
M5224 nw671 t1938 vdd vdd pch w=2u l=180n
CT1942 t1942 0 0.1f
M5225 nw671 t1937 t1942 0 nch w=1u l=180n
M5226 t1942 t1938 0 0 nch w=1u l=180n
Cnw671 nw671 0 2f
CT1943 t1943 0 0.1f
CT1944 t1944 0 0.1f
CT1945 t1945 0 0.1f
M5227 t1943 nw671 vdd vdd pch w=2u l=180n
M5228 t1943 nw670 vdd vdd pch w=2u l=180n
CT1946 t1946 0 0.1f
M5229 t1943 nw671 t1946 0 nch w=1u l=180n
M5230 t1946 nw670 0 0 nch w=1u l=180n
M5231 t1944 nw671 vdd vdd pch w=2u l=180n
M5232 t1944 t1943 vdd vdd pch w=2u l=180n
CT1947 t1947 0 0.1f
M5233 t1944 nw671 t1947 0 nch w=1u l=180n
M5234 t1947 t1943 0 0 nch w=1u l=180n
M5235 t1945 nw670 vdd vdd pch w=2u l=180n
M5236 t1945 t1943 vdd vdd pch w=2u l=180n
CT1948 t1948 0 0.1f
M5237 t1945 nw670 t1948 0 nch w=1u l=180n
M5238 t1948 t1943 0 0 nch w=1u l=180n
M5239 nw672 t1944 vdd vdd pch w=2u l=180n
M5240 nw672 t1945 vdd vdd pch w=2u l=180n
CT1949 t1949 0 0.1f
M5241 nw672 t1944 t1949 0 nch w=1u l=180n
M5242 t1949 t1945 0 0 nch w=1u l=180n
Cnw672 nw672 0 2f
M5243 nw673 nw104 vdd vdd pch w=2u l=180n
M5244 nw673 nw600 vdd vdd pch w=2u l=180n
CT1950 t1950 0 0.1f
M5245 nw673 nw104 t1950 0 nch w=1u l=180n
M5246 t1950 nw600 0 0 nch w=1u l=180n
Cnw673 nw673 0 2f
M5247 nw674 nw671 vdd vdd pch w=2u l=180n
M5248 nw674 nw670 vdd vdd pch w=2u l=180n
CT1951 t1951 0 0.1f
M5249 nw674 nw671 t1951 0 nch w=1u l=180n
M5250 t1951 nw670 0 0 nch w=1u l=180n
Cnw674 nw674 0 2f
M5251 nw675 nw673 vdd vdd pch w=2u l=180n
M5252 nw675 nw674 vdd vdd pch w=2u l=180n
CT1952 t1952 0 0.1f
M5253 nw675 nw673 t1952 0 nch w=1u l=180n
M5254 t1952 nw674 0 0 nch w=1u l=180n
Cnw675 nw675 0 2f
CT1953 t1953 0 0.1f
CT1954 t1954 0 0.1f
CT1955 t1955 0 0.1f
M5255 t1953 nw105 vdd vdd pch w=2u l=180n
M5256 t1953 nw605 vdd vdd pch w=2u l=180n
CT1956 t1956 0 0.1f
M5257 t1953 nw105 t1956 0 nch w=1u l=180n
M5258 t1956 nw605 0 0 nch w=1u l=180n
M5259 t1954 nw105 vdd vdd pch w=2u l=180n
M5260 t1954 t1953 vdd vdd pch w=2u l=180n
CT1957 t1957 0 0.1f
M5261 t1954 nw105 t1957 0 nch w=1u l=180n
M5262 t1957 t1953 0 0 nch w=1u l=180n
M5263 t1955 nw605 vdd vdd pch w=2u l=180n
M5264 t1955 t1953 vdd vdd pch w=2u l=180n
CT1958 t1958 0 0.1f
M5265 t1955 nw605 t1958 0 nch w=1u l=180n
M5266 t1958 t1953 0 0 nch w=1u l=180n
M5267 nw676 t1954 vdd vdd pch w=2u l=180n
M5268 nw676 t1955 vdd vdd pch w=2u l=180n
CT1959 t1959 0 0.1f
M5269 nw676 t1954 t1959 0 nch w=1u l=180n
M5270 t1959 t1955 0 0 nch w=1u l=180n
Cnw676 nw676 0 2f
CT1960 t1960 0 0.1f
CT1961 t1961 0 0.1f
CT1962 t1962 0 0.1f
M5271 t1960 nw676 vdd vdd pch w=2u l=180n
M5272 t1960 nw675 vdd vdd pch w=2u l=180n
CT1963 t1963 0 0.1f
M5273 t1960 nw676 t1963 0 nch w=1u l=180n
M5274 t1963 nw675 0 0 nch w=1u l=180n
M5275 t1961 nw676 vdd vdd pch w=2u l=180n
M5276 t1961 t1960 vdd vdd pch w=2u l=180n
CT1964 t1964 0 0.1f
M5277 t1961 nw676 t1964 0 nch w=1u l=180n
M5278 t1964 t1960 0 0 nch w=1u l=180n
M5279 t1962 nw675 vdd vdd pch w=2u l=180n
M5280 t1962 t1960 vdd vdd pch w=2u l=180n
CT1965 t1965 0 0.1f
M5281 t1962 nw675 t1965 0 nch w=1u l=180n
M5282 t1965 t1960 0 0 nch w=1u l=180n
M5283 nw677 t1961 vdd vdd pch w=2u l=180n
M5284 nw677 t1962 vdd vdd pch w=2u l=180n
CT1966 t1966 0 0.1f
M5285 nw677 t1961 t1966 0 nch w=1u l=180n
M5286 t1966 t1962 0 0 nch w=1u l=180n
Cnw677 nw677 0 2f
M5287 nw678 nw105 vdd vdd pch w=2u l=180n
M5288 nw678 nw605 vdd vdd pch w=2u l=180n
CT1967 t1967 0 0.1f
M5289 nw678 nw105 t1967 0 nch w=1u l=180n
M5290 t1967 nw605 0 0 nch w=1u l=180n
Cnw678 nw678 0 2f
M5291 nw679 nw676 vdd vdd pch w=2u l=180n
M5292 nw679 nw675 vdd vdd pch w=2u l=180n
CT1968 t1968 0 0.1f
M5293 nw679 nw676 t1968 0 nch w=1u l=180n
M5294 t1968 nw675 0 0 nch w=1u l=180n
Cnw679 nw679 0 2f
M5295 nw680 nw678 vdd vdd pch w=2u l=180n
M5296 nw680 nw679 vdd vdd pch w=2u l=180n
CT1969 t1969 0 0.1f
M5297 nw680 nw678 t1969 0 nch w=1u l=180n
M5298 t1969 nw679 0 0 nch w=1u l=180n
Cnw680 nw680 0 2f
CT1970 t1970 0 0.1f
CT1971 t1971 0 0.1f
CT1972 t1972 0 0.1f
M5299 t1970 nw106 vdd vdd pch w=2u l=180n
M5300 t1970 nw610 vdd vdd pch w=2u l=180n
CT1973 t1973 0 0.1f
M5301 t1970 nw106 t1973 0 nch w=1u l=180n
M5302 t1973 nw610 0 0 nch w=1u l=180n
M5303 t1971 nw106 vdd vdd pch w=2u l=180n
M5304 t1971 t1970 vdd vdd pch w=2u l=180n
CT1974 t1974 0 0.1f
M5305 t1971 nw106 t1974 0 nch w=1u l=180n
M5306 t1974 t1970 0 0 nch w=1u l=180n
M5307 t1972 nw610 vdd vdd pch w=2u l=180n
M5308 t1972 t1970 vdd vdd pch w=2u l=180n
CT1975 t1975 0 0.1f
M5309 t1972 nw610 t1975 0 nch w=1u l=180n
M5310 t1975 t1970 0 0 nch w=1u l=180n
M5311 nw681 t1971 vdd vdd pch w=2u l=180n
M5312 nw681 t1972 vdd vdd pch w=2u l=180n
CT1976 t1976 0 0.1f
M5313 nw681 t1971 t1976 0 nch w=1u l=180n
M5314 t1976 t1972 0 0 nch w=1u l=180n
Cnw681 nw681 0 2f
CT1977 t1977 0 0.1f
CT1978 t1978 0 0.1f
CT1979 t1979 0 0.1f
M5315 t1977 nw681 vdd vdd pch w=2u l=180n
M5316 t1977 nw680 vdd vdd pch w=2u l=180n
CT1980 t1980 0 0.1f
M5317 t1977 nw681 t1980 0 nch w=1u l=180n
M5318 t1980 nw680 0 0 nch w=1u l=180n
M5319 t1978 nw681 vdd vdd pch w=2u l=180n
M5320 t1978 t1977 vdd vdd pch w=2u l=180n
CT1981 t1981 0 0.1f
M5321 t1978 nw681 t1981 0 nch w=1u l=180n
M5322 t1981 t1977 0 0 nch w=1u l=180n
M5323 t1979 nw680 vdd vdd pch w=2u l=180n
M5324 t1979 t1977 vdd vdd pch w=2u l=180n
CT1982 t1982 0 0.1f
M5325 t1979 nw680 t1982 0 nch w=1u l=180n
M5326 t1982 t1977 0 0 nch w=1u l=180n
M5327 nw682 t1978 vdd vdd pch w=2u l=180n
M5328 nw682 t1979 vdd vdd pch w=2u l=180n
CT1983 t1983 0 0.1f
M5329 nw682 t1978 t1983 0 nch w=1u l=180n
M5330 t1983 t1979 0 0 nch w=1u l=180n
Cnw682 nw682 0 2f
M5331 nw683 nw106 vdd vdd pch w=2u l=180n
M5332 nw683 nw610 vdd vdd pch w=2u l=180n
CT1984 t1984 0 0.1f
M5333 nw683 nw106 t1984 0 nch w=1u l=180n
M5334 t1984 nw610 0 0 nch w=1u l=180n
Cnw683 nw683 0 2f
M5335 nw684 nw681 vdd vdd pch w=2u l=180n
M5336 nw684 nw680 vdd vdd pch w=2u l=180n
CT1985 t1985 0 0.1f
M5337 nw684 nw681 t1985 0 nch w=1u l=180n
M5338 t1985 nw680 0 0 nch w=1u l=180n
Cnw684 nw684 0 2f
M5339 nw685 nw683 vdd vdd pch w=2u l=180n
M5340 nw685 nw684 vdd vdd pch w=2u l=180n
CT1986 t1986 0 0.1f
M5341 nw685 nw683 t1986 0 nch w=1u l=180n
M5342 t1986 nw684 0 0 nch w=1u l=180n
Cnw685 nw685 0 2f
CT1987 t1987 0 0.1f
CT1988 t1988 0 0.1f
CT1989 t1989 0 0.1f
M5343 t1987 nw107 vdd vdd pch w=2u l=180n
M5344 t1987 nw615 vdd vdd pch w=2u l=180n
CT1990 t1990 0 0.1f
M5345 t1987 nw107 t1990 0 nch w=1u l=180n
M5346 t1990 nw615 0 0 nch w=1u l=180n
M5347 t1988 nw107 vdd vdd pch w=2u l=180n
M5348 t1988 t1987 vdd vdd pch w=2u l=180n
CT1991 t1991 0 0.1f
M5349 t1988 nw107 t1991 0 nch w=1u l=180n
M5350 t1991 t1987 0 0 nch w=1u l=180n
M5351 t1989 nw615 vdd vdd pch w=2u l=180n
M5352 t1989 t1987 vdd vdd pch w=2u l=180n
CT1992 t1992 0 0.1f
M5353 t1989 nw615 t1992 0 nch w=1u l=180n
M5354 t1992 t1987 0 0 nch w=1u l=180n
M5355 nw686 t1988 vdd vdd pch w=2u l=180n
M5356 nw686 t1989 vdd vdd pch w=2u l=180n
CT1993 t1993 0 0.1f
M5357 nw686 t1988 t1993 0 nch w=1u l=180n
M5358 t1993 t1989 0 0 nch w=1u l=180n
Cnw686 nw686 0 2f
CT1994 t1994 0 0.1f
CT1995 t1995 0 0.1f
CT1996 t1996 0 0.1f
M5359 t1994 nw686 vdd vdd pch w=2u l=180n
M5360 t1994 nw685 vdd vdd pch w=2u l=180n
CT1997 t1997 0 0.1f
M5361 t1994 nw686 t1997 0 nch w=1u l=180n
M5362 t1997 nw685 0 0 nch w=1u l=180n
M5363 t1995 nw686 vdd vdd pch w=2u l=180n
M5364 t1995 t1994 vdd vdd pch w=2u l=180n
CT1998 t1998 0 0.1f
M5365 t1995 nw686 t1998 0 nch w=1u l=180n
M5366 t1998 t1994 0 0 nch w=1u l=180n
M5367 t1996 nw685 vdd vdd pch w=2u l=180n
M5368 t1996 t1994 vdd vdd pch w=2u l=180n
CT1999 t1999 0 0.1f
M5369 t1996 nw685 t1999 0 nch w=1u l=180n
M5370 t1999 t1994 0 0 nch w=1u l=180n
M5371 nw687 t1995 vdd vdd pch w=2u l=180n
M5372 nw687 t1996 vdd vdd pch w=2u l=180n
CT2000 t2000 0 0.1f
M5373 nw687 t1995 t2000 0 nch w=1u l=180n
M5374 t2000 t1996 0 0 nch w=1u l=180n
Cnw687 nw687 0 2f
M5375 nw688 nw107 vdd vdd pch w=2u l=180n
M5376 nw688 nw615 vdd vdd pch w=2u l=180n
CT2001 t2001 0 0.1f
M5377 nw688 nw107 t2001 0 nch w=1u l=180n
M5378 t2001 nw615 0 0 nch w=1u l=180n
Cnw688 nw688 0 2f
M5379 nw689 nw686 vdd vdd pch w=2u l=180n
M5380 nw689 nw685 vdd vdd pch w=2u l=180n
CT2002 t2002 0 0.1f
M5381 nw689 nw686 t2002 0 nch w=1u l=180n
M5382 t2002 nw685 0 0 nch w=1u l=180n
Cnw689 nw689 0 2f
M5383 nw690 nw688 vdd vdd pch w=2u l=180n
M5384 nw690 nw689 vdd vdd pch w=2u l=180n
CT2003 t2003 0 0.1f
M5385 nw690 nw688 t2003 0 nch w=1u l=180n
M5386 t2003 nw689 0 0 nch w=1u l=180n
Cnw690 nw690 0 2f
CT2004 t2004 0 0.1f
CT2005 t2005 0 0.1f
CT2006 t2006 0 0.1f
M5387 t2004 nw108 vdd vdd pch w=2u l=180n
M5388 t2004 nw620 vdd vdd pch w=2u l=180n
CT2007 t2007 0 0.1f
M5389 t2004 nw108 t2007 0 nch w=1u l=180n
M5390 t2007 nw620 0 0 nch w=1u l=180n
M5391 t2005 nw108 vdd vdd pch w=2u l=180n
M5392 t2005 t2004 vdd vdd pch w=2u l=180n
CT2008 t2008 0 0.1f
M5393 t2005 nw108 t2008 0 nch w=1u l=180n
M5394 t2008 t2004 0 0 nch w=1u l=180n
M5395 t2006 nw620 vdd vdd pch w=2u l=180n
M5396 t2006 t2004 vdd vdd pch w=2u l=180n
CT2009 t2009 0 0.1f
M5397 t2006 nw620 t2009 0 nch w=1u l=180n
M5398 t2009 t2004 0 0 nch w=1u l=180n
M5399 nw691 t2005 vdd vdd pch w=2u l=180n
M5400 nw691 t2006 vdd vdd pch w=2u l=180n
CT2010 t2010 0 0.1f
M5401 nw691 t2005 t2010 0 nch w=1u l=180n
M5402 t2010 t2006 0 0 nch w=1u l=180n
Cnw691 nw691 0 2f
CT2011 t2011 0 0.1f
CT2012 t2012 0 0.1f
CT2013 t2013 0 0.1f
M5403 t2011 nw691 vdd vdd pch w=2u l=180n
M5404 t2011 nw690 vdd vdd pch w=2u l=180n
CT2014 t2014 0 0.1f
M5405 t2011 nw691 t2014 0 nch w=1u l=180n
M5406 t2014 nw690 0 0 nch w=1u l=180n
M5407 t2012 nw691 vdd vdd pch w=2u l=180n
M5408 t2012 t2011 vdd vdd pch w=2u l=180n
CT2015 t2015 0 0.1f
M5409 t2012 nw691 t2015 0 nch w=1u l=180n
M5410 t2015 t2011 0 0 nch w=1u l=180n
M5411 t2013 nw690 vdd vdd pch w=2u l=180n
M5412 t2013 t2011 vdd vdd pch w=2u l=180n
CT2016 t2016 0 0.1f
M5413 t2013 nw690 t2016 0 nch w=1u l=180n
M5414 t2016 t2011 0 0 nch w=1u l=180n
M5415 nw692 t2012 vdd vdd pch w=2u l=180n
M5416 nw692 t2013 vdd vdd pch w=2u l=180n
CT2017 t2017 0 0.1f
M5417 nw692 t2012 t2017 0 nch w=1u l=180n
M5418 t2017 t2013 0 0 nch w=1u l=180n
Cnw692 nw692 0 2f
M5419 nw693 nw108 vdd vdd pch w=2u l=180n
M5420 nw693 nw620 vdd vdd pch w=2u l=180n
CT2018 t2018 0 0.1f
M5421 nw693 nw108 t2018 0 nch w=1u l=180n
M5422 t2018 nw620 0 0 nch w=1u l=180n
Cnw693 nw693 0 2f
M5423 nw694 nw691 vdd vdd pch w=2u l=180n
M5424 nw694 nw690 vdd vdd pch w=2u l=180n
CT2019 t2019 0 0.1f
M5425 nw694 nw691 t2019 0 nch w=1u l=180n
M5426 t2019 nw690 0 0 nch w=1u l=180n
Cnw694 nw694 0 2f
M5427 nw695 nw693 vdd vdd pch w=2u l=180n
M5428 nw695 nw694 vdd vdd pch w=2u l=180n
CT2020 t2020 0 0.1f
M5429 nw695 nw693 t2020 0 nch w=1u l=180n
M5430 t2020 nw694 0 0 nch w=1u l=180n
Cnw695 nw695 0 2f
CT2021 t2021 0 0.1f
CT2022 t2022 0 0.1f
CT2023 t2023 0 0.1f
M5431 t2021 nw109 vdd vdd pch w=2u l=180n
M5432 t2021 nw625 vdd vdd pch w=2u l=180n
CT2024 t2024 0 0.1f
M5433 t2021 nw109 t2024 0 nch w=1u l=180n
M5434 t2024 nw625 0 0 nch w=1u l=180n
M5435 t2022 nw109 vdd vdd pch w=2u l=180n
M5436 t2022 t2021 vdd vdd pch w=2u l=180n
CT2025 t2025 0 0.1f
M5437 t2022 nw109 t2025 0 nch w=1u l=180n
M5438 t2025 t2021 0 0 nch w=1u l=180n
M5439 t2023 nw625 vdd vdd pch w=2u l=180n
M5440 t2023 t2021 vdd vdd pch w=2u l=180n
CT2026 t2026 0 0.1f
M5441 t2023 nw625 t2026 0 nch w=1u l=180n
M5442 t2026 t2021 0 0 nch w=1u l=180n
M5443 nw696 t2022 vdd vdd pch w=2u l=180n
M5444 nw696 t2023 vdd vdd pch w=2u l=180n
CT2027 t2027 0 0.1f
M5445 nw696 t2022 t2027 0 nch w=1u l=180n
M5446 t2027 t2023 0 0 nch w=1u l=180n
Cnw696 nw696 0 2f
CT2028 t2028 0 0.1f
CT2029 t2029 0 0.1f
CT2030 t2030 0 0.1f
M5447 t2028 nw696 vdd vdd pch w=2u l=180n
M5448 t2028 nw695 vdd vdd pch w=2u l=180n
CT2031 t2031 0 0.1f
M5449 t2028 nw696 t2031 0 nch w=1u l=180n
M5450 t2031 nw695 0 0 nch w=1u l=180n
M5451 t2029 nw696 vdd vdd pch w=2u l=180n
M5452 t2029 t2028 vdd vdd pch w=2u l=180n
CT2032 t2032 0 0.1f
M5453 t2029 nw696 t2032 0 nch w=1u l=180n
M5454 t2032 t2028 0 0 nch w=1u l=180n
M5455 t2030 nw695 vdd vdd pch w=2u l=180n
M5456 t2030 t2028 vdd vdd pch w=2u l=180n
CT2033 t2033 0 0.1f
M5457 t2030 nw695 t2033 0 nch w=1u l=180n
M5458 t2033 t2028 0 0 nch w=1u l=180n
M5459 nw697 t2029 vdd vdd pch w=2u l=180n
M5460 nw697 t2030 vdd vdd pch w=2u l=180n
CT2034 t2034 0 0.1f
M5461 nw697 t2029 t2034 0 nch w=1u l=180n
M5462 t2034 t2030 0 0 nch w=1u l=180n
Cnw697 nw697 0 2f
M5463 nw698 nw109 vdd vdd pch w=2u l=180n
M5464 nw698 nw625 vdd vdd pch w=2u l=180n
CT2035 t2035 0 0.1f
M5465 nw698 nw109 t2035 0 nch w=1u l=180n
M5466 t2035 nw625 0 0 nch w=1u l=180n
Cnw698 nw698 0 2f
M5467 nw699 nw696 vdd vdd pch w=2u l=180n
M5468 nw699 nw695 vdd vdd pch w=2u l=180n
CT2036 t2036 0 0.1f
M5469 nw699 nw696 t2036 0 nch w=1u l=180n
M5470 t2036 nw695 0 0 nch w=1u l=180n
Cnw699 nw699 0 2f
M5471 nw700 nw698 vdd vdd pch w=2u l=180n
M5472 nw700 nw699 vdd vdd pch w=2u l=180n
CT2037 t2037 0 0.1f
M5473 nw700 nw698 t2037 0 nch w=1u l=180n
M5474 t2037 nw699 0 0 nch w=1u l=180n
Cnw700 nw700 0 2f
CT2038 t2038 0 0.1f
CT2039 t2039 0 0.1f
CT2040 t2040 0 0.1f
M5475 t2038 nw110 vdd vdd pch w=2u l=180n
M5476 t2038 nw630 vdd vdd pch w=2u l=180n
CT2041 t2041 0 0.1f
M5477 t2038 nw110 t2041 0 nch w=1u l=180n
M5478 t2041 nw630 0 0 nch w=1u l=180n
M5479 t2039 nw110 vdd vdd pch w=2u l=180n
M5480 t2039 t2038 vdd vdd pch w=2u l=180n
CT2042 t2042 0 0.1f
M5481 t2039 nw110 t2042 0 nch w=1u l=180n
M5482 t2042 t2038 0 0 nch w=1u l=180n
M5483 t2040 nw630 vdd vdd pch w=2u l=180n
M5484 t2040 t2038 vdd vdd pch w=2u l=180n
CT2043 t2043 0 0.1f
M5485 t2040 nw630 t2043 0 nch w=1u l=180n
M5486 t2043 t2038 0 0 nch w=1u l=180n
M5487 nw701 t2039 vdd vdd pch w=2u l=180n
M5488 nw701 t2040 vdd vdd pch w=2u l=180n
CT2044 t2044 0 0.1f
M5489 nw701 t2039 t2044 0 nch w=1u l=180n
M5490 t2044 t2040 0 0 nch w=1u l=180n
Cnw701 nw701 0 2f
CT2045 t2045 0 0.1f
CT2046 t2046 0 0.1f
CT2047 t2047 0 0.1f
M5491 t2045 nw701 vdd vdd pch w=2u l=180n
M5492 t2045 nw700 vdd vdd pch w=2u l=180n
CT2048 t2048 0 0.1f
M5493 t2045 nw701 t2048 0 nch w=1u l=180n
M5494 t2048 nw700 0 0 nch w=1u l=180n
M5495 t2046 nw701 vdd vdd pch w=2u l=180n
M5496 t2046 t2045 vdd vdd pch w=2u l=180n
CT2049 t2049 0 0.1f
M5497 t2046 nw701 t2049 0 nch w=1u l=180n
M5498 t2049 t2045 0 0 nch w=1u l=180n
M5499 t2047 nw700 vdd vdd pch w=2u l=180n
M5500 t2047 t2045 vdd vdd pch w=2u l=180n
CT2050 t2050 0 0.1f
M5501 t2047 nw700 t2050 0 nch w=1u l=180n
M5502 t2050 t2045 0 0 nch w=1u l=180n
M5503 nw702 t2046 vdd vdd pch w=2u l=180n
M5504 nw702 t2047 vdd vdd pch w=2u l=180n
CT2051 t2051 0 0.1f
M5505 nw702 t2046 t2051 0 nch w=1u l=180n
M5506 t2051 t2047 0 0 nch w=1u l=180n
Cnw702 nw702 0 2f
M5507 nw703 nw110 vdd vdd pch w=2u l=180n
M5508 nw703 nw630 vdd vdd pch w=2u l=180n
CT2052 t2052 0 0.1f
M5509 nw703 nw110 t2052 0 nch w=1u l=180n
M5510 t2052 nw630 0 0 nch w=1u l=180n
Cnw703 nw703 0 2f
M5511 nw704 nw701 vdd vdd pch w=2u l=180n
M5512 nw704 nw700 vdd vdd pch w=2u l=180n
CT2053 t2053 0 0.1f
M5513 nw704 nw701 t2053 0 nch w=1u l=180n
M5514 t2053 nw700 0 0 nch w=1u l=180n
Cnw704 nw704 0 2f
M5515 nw705 nw703 vdd vdd pch w=2u l=180n
M5516 nw705 nw704 vdd vdd pch w=2u l=180n
CT2054 t2054 0 0.1f
M5517 nw705 nw703 t2054 0 nch w=1u l=180n
M5518 t2054 nw704 0 0 nch w=1u l=180n
Cnw705 nw705 0 2f
CT2055 t2055 0 0.1f
CT2056 t2056 0 0.1f
CT2057 t2057 0 0.1f
M5519 t2055 nw111 vdd vdd pch w=2u l=180n
M5520 t2055 nw635 vdd vdd pch w=2u l=180n
CT2058 t2058 0 0.1f
M5521 t2055 nw111 t2058 0 nch w=1u l=180n
M5522 t2058 nw635 0 0 nch w=1u l=180n
M5523 t2056 nw111 vdd vdd pch w=2u l=180n
M5524 t2056 t2055 vdd vdd pch w=2u l=180n
CT2059 t2059 0 0.1f
M5525 t2056 nw111 t2059 0 nch w=1u l=180n
M5526 t2059 t2055 0 0 nch w=1u l=180n
M5527 t2057 nw635 vdd vdd pch w=2u l=180n
M5528 t2057 t2055 vdd vdd pch w=2u l=180n
CT2060 t2060 0 0.1f
M5529 t2057 nw635 t2060 0 nch w=1u l=180n
M5530 t2060 t2055 0 0 nch w=1u l=180n
M5531 nw706 t2056 vdd vdd pch w=2u l=180n
M5532 nw706 t2057 vdd vdd pch w=2u l=180n
CT2061 t2061 0 0.1f
M5533 nw706 t2056 t2061 0 nch w=1u l=180n
M5534 t2061 t2057 0 0 nch w=1u l=180n
Cnw706 nw706 0 2f
CT2062 t2062 0 0.1f
CT2063 t2063 0 0.1f
CT2064 t2064 0 0.1f
M5535 t2062 nw706 vdd vdd pch w=2u l=180n
M5536 t2062 nw705 vdd vdd pch w=2u l=180n
CT2065 t2065 0 0.1f
M5537 t2062 nw706 t2065 0 nch w=1u l=180n
M5538 t2065 nw705 0 0 nch w=1u l=180n
M5539 t2063 nw706 vdd vdd pch w=2u l=180n
M5540 t2063 t2062 vdd vdd pch w=2u l=180n
CT2066 t2066 0 0.1f
M5541 t2063 nw706 t2066 0 nch w=1u l=180n
M5542 t2066 t2062 0 0 nch w=1u l=180n
M5543 t2064 nw705 vdd vdd pch w=2u l=180n
M5544 t2064 t2062 vdd vdd pch w=2u l=180n
CT2067 t2067 0 0.1f
M5545 t2064 nw705 t2067 0 nch w=1u l=180n
M5546 t2067 t2062 0 0 nch w=1u l=180n
M5547 nw707 t2063 vdd vdd pch w=2u l=180n
M5548 nw707 t2064 vdd vdd pch w=2u l=180n
CT2068 t2068 0 0.1f
M5549 nw707 t2063 t2068 0 nch w=1u l=180n
M5550 t2068 t2064 0 0 nch w=1u l=180n
Cnw707 nw707 0 2f
M5551 nw708 nw111 vdd vdd pch w=2u l=180n
M5552 nw708 nw635 vdd vdd pch w=2u l=180n
CT2069 t2069 0 0.1f
M5553 nw708 nw111 t2069 0 nch w=1u l=180n
M5554 t2069 nw635 0 0 nch w=1u l=180n
Cnw708 nw708 0 2f
M5555 nw709 nw706 vdd vdd pch w=2u l=180n
M5556 nw709 nw705 vdd vdd pch w=2u l=180n
CT2070 t2070 0 0.1f
M5557 nw709 nw706 t2070 0 nch w=1u l=180n
M5558 t2070 nw705 0 0 nch w=1u l=180n
Cnw709 nw709 0 2f
M5559 nw710 nw708 vdd vdd pch w=2u l=180n
M5560 nw710 nw709 vdd vdd pch w=2u l=180n
CT2071 t2071 0 0.1f
M5561 nw710 nw708 t2071 0 nch w=1u l=180n
M5562 t2071 nw709 0 0 nch w=1u l=180n
Cnw710 nw710 0 2f
CT2072 t2072 0 0.1f
CT2073 t2073 0 0.1f
CT2074 t2074 0 0.1f
M5563 t2072 nw112 vdd vdd pch w=2u l=180n
M5564 t2072 nw638 vdd vdd pch w=2u l=180n
CT2075 t2075 0 0.1f
M5565 t2072 nw112 t2075 0 nch w=1u l=180n
M5566 t2075 nw638 0 0 nch w=1u l=180n
M5567 t2073 nw112 vdd vdd pch w=2u l=180n
M5568 t2073 t2072 vdd vdd pch w=2u l=180n
CT2076 t2076 0 0.1f
M5569 t2073 nw112 t2076 0 nch w=1u l=180n
M5570 t2076 t2072 0 0 nch w=1u l=180n
M5571 t2074 nw638 vdd vdd pch w=2u l=180n
M5572 t2074 t2072 vdd vdd pch w=2u l=180n
CT2077 t2077 0 0.1f
M5573 t2074 nw638 t2077 0 nch w=1u l=180n
M5574 t2077 t2072 0 0 nch w=1u l=180n
M5575 nw711 t2073 vdd vdd pch w=2u l=180n
M5576 nw711 t2074 vdd vdd pch w=2u l=180n
CT2078 t2078 0 0.1f
M5577 nw711 t2073 t2078 0 nch w=1u l=180n
M5578 t2078 t2074 0 0 nch w=1u l=180n
Cnw711 nw711 0 2f
CT2079 t2079 0 0.1f
CT2080 t2080 0 0.1f
CT2081 t2081 0 0.1f
M5579 t2079 nw711 vdd vdd pch w=2u l=180n
M5580 t2079 nw710 vdd vdd pch w=2u l=180n
CT2082 t2082 0 0.1f
M5581 t2079 nw711 t2082 0 nch w=1u l=180n
M5582 t2082 nw710 0 0 nch w=1u l=180n
M5583 t2080 nw711 vdd vdd pch w=2u l=180n
M5584 t2080 t2079 vdd vdd pch w=2u l=180n
CT2083 t2083 0 0.1f
M5585 t2080 nw711 t2083 0 nch w=1u l=180n
M5586 t2083 t2079 0 0 nch w=1u l=180n
M5587 t2081 nw710 vdd vdd pch w=2u l=180n
M5588 t2081 t2079 vdd vdd pch w=2u l=180n
CT2084 t2084 0 0.1f
M5589 t2081 nw710 t2084 0 nch w=1u l=180n
M5590 t2084 t2079 0 0 nch w=1u l=180n
M5591 nw712 t2080 vdd vdd pch w=2u l=180n
M5592 nw712 t2081 vdd vdd pch w=2u l=180n
CT2085 t2085 0 0.1f
M5593 nw712 t2080 t2085 0 nch w=1u l=180n
M5594 t2085 t2081 0 0 nch w=1u l=180n
Cnw712 nw712 0 2f
M5595 nw713 nw112 vdd vdd pch w=2u l=180n
M5596 nw713 nw638 vdd vdd pch w=2u l=180n
CT2086 t2086 0 0.1f
M5597 nw713 nw112 t2086 0 nch w=1u l=180n
M5598 t2086 nw638 0 0 nch w=1u l=180n
Cnw713 nw713 0 2f
M5599 nw714 nw711 vdd vdd pch w=2u l=180n
M5600 nw714 nw710 vdd vdd pch w=2u l=180n
CT2087 t2087 0 0.1f
M5601 nw714 nw711 t2087 0 nch w=1u l=180n
M5602 t2087 nw710 0 0 nch w=1u l=180n
Cnw714 nw714 0 2f
M5603 nw715 nw713 vdd vdd pch w=2u l=180n
M5604 nw715 nw714 vdd vdd pch w=2u l=180n
CT2088 t2088 0 0.1f
M5605 nw715 nw713 t2088 0 nch w=1u l=180n
M5606 t2088 nw714 0 0 nch w=1u l=180n
Cnw715 nw715 0 2f
CT2089 t2089 0 0.1f
CT2090 t2090 0 0.1f
CT2091 t2091 0 0.1f
M5607 t2089 nw113 vdd vdd pch w=2u l=180n
M5608 t2089 nw642 vdd vdd pch w=2u l=180n
CT2092 t2092 0 0.1f
M5609 t2089 nw113 t2092 0 nch w=1u l=180n
M5610 t2092 nw642 0 0 nch w=1u l=180n
M5611 t2090 nw113 vdd vdd pch w=2u l=180n
M5612 t2090 t2089 vdd vdd pch w=2u l=180n
CT2093 t2093 0 0.1f
M5613 t2090 nw113 t2093 0 nch w=1u l=180n
M5614 t2093 t2089 0 0 nch w=1u l=180n
M5615 t2091 nw642 vdd vdd pch w=2u l=180n
M5616 t2091 t2089 vdd vdd pch w=2u l=180n
CT2094 t2094 0 0.1f
M5617 t2091 nw642 t2094 0 nch w=1u l=180n
M5618 t2094 t2089 0 0 nch w=1u l=180n
M5619 nw716 t2090 vdd vdd pch w=2u l=180n
M5620 nw716 t2091 vdd vdd pch w=2u l=180n
CT2095 t2095 0 0.1f
M5621 nw716 t2090 t2095 0 nch w=1u l=180n
M5622 t2095 t2091 0 0 nch w=1u l=180n
Cnw716 nw716 0 2f
CT2096 t2096 0 0.1f
M5623 t2096 nw113 vdd vdd pch w=2u l=180n
M5624 t2096 nw642 vdd vdd pch w=2u l=180n
CT2097 t2097 0 0.1f
M5625 t2096 nw113 t2097 0 nch w=1u l=180n
M5626 t2097 nw642 0 0 nch w=1u l=180n
M5627 nw717 t2096 vdd vdd pch w=2u l=180n
M5628 nw717 t2096 0 0 nch w=1u l=180n
Cnw717 nw717 0 2f
CT2098 t2098 0 0.1f
CT2099 t2099 0 0.1f
CT2100 t2100 0 0.1f
M5629 t2098 nw114 vdd vdd pch w=2u l=180n
M5630 t2098 nw647 vdd vdd pch w=2u l=180n
CT2101 t2101 0 0.1f
M5631 t2098 nw114 t2101 0 nch w=1u l=180n
M5632 t2101 nw647 0 0 nch w=1u l=180n
M5633 t2099 nw114 vdd vdd pch w=2u l=180n
M5634 t2099 t2098 vdd vdd pch w=2u l=180n
CT2102 t2102 0 0.1f
M5635 t2099 nw114 t2102 0 nch w=1u l=180n
M5636 t2102 t2098 0 0 nch w=1u l=180n
M5637 t2100 nw647 vdd vdd pch w=2u l=180n
M5638 t2100 t2098 vdd vdd pch w=2u l=180n
CT2103 t2103 0 0.1f
M5639 t2100 nw647 t2103 0 nch w=1u l=180n
M5640 t2103 t2098 0 0 nch w=1u l=180n
M5641 nw718 t2099 vdd vdd pch w=2u l=180n
M5642 nw718 t2100 vdd vdd pch w=2u l=180n
CT2104 t2104 0 0.1f
M5643 nw718 t2099 t2104 0 nch w=1u l=180n
M5644 t2104 t2100 0 0 nch w=1u l=180n
Cnw718 nw718 0 2f
CT2105 t2105 0 0.1f
CT2106 t2106 0 0.1f
CT2107 t2107 0 0.1f
M5645 t2105 nw718 vdd vdd pch w=2u l=180n
M5646 t2105 nw717 vdd vdd pch w=2u l=180n
CT2108 t2108 0 0.1f
M5647 t2105 nw718 t2108 0 nch w=1u l=180n
M5648 t2108 nw717 0 0 nch w=1u l=180n
M5649 t2106 nw718 vdd vdd pch w=2u l=180n
M5650 t2106 t2105 vdd vdd pch w=2u l=180n
CT2109 t2109 0 0.1f
M5651 t2106 nw718 t2109 0 nch w=1u l=180n
M5652 t2109 t2105 0 0 nch w=1u l=180n
M5653 t2107 nw717 vdd vdd pch w=2u l=180n
M5654 t2107 t2105 vdd vdd pch w=2u l=180n
CT2110 t2110 0 0.1f
M5655 t2107 nw717 t2110 0 nch w=1u l=180n
M5656 t2110 t2105 0 0 nch w=1u l=180n
M5657 nw719 t2106 vdd vdd pch w=2u l=180n
M5658 nw719 t2107 vdd vdd pch w=2u l=180n
CT2111 t2111 0 0.1f
M5659 nw719 t2106 t2111 0 nch w=1u l=180n
M5660 t2111 t2107 0 0 nch w=1u l=180n
Cnw719 nw719 0 2f
M5661 nw720 nw114 vdd vdd pch w=2u l=180n
M5662 nw720 nw647 vdd vdd pch w=2u l=180n
CT2112 t2112 0 0.1f
M5663 nw720 nw114 t2112 0 nch w=1u l=180n
M5664 t2112 nw647 0 0 nch w=1u l=180n
Cnw720 nw720 0 2f
M5665 nw721 nw718 vdd vdd pch w=2u l=180n
M5666 nw721 nw717 vdd vdd pch w=2u l=180n
CT2113 t2113 0 0.1f
M5667 nw721 nw718 t2113 0 nch w=1u l=180n
M5668 t2113 nw717 0 0 nch w=1u l=180n
Cnw721 nw721 0 2f
M5669 nw722 nw720 vdd vdd pch w=2u l=180n
M5670 nw722 nw721 vdd vdd pch w=2u l=180n
CT2114 t2114 0 0.1f
M5671 nw722 nw720 t2114 0 nch w=1u l=180n
M5672 t2114 nw721 0 0 nch w=1u l=180n
Cnw722 nw722 0 2f
CT2115 t2115 0 0.1f
CT2116 t2116 0 0.1f
CT2117 t2117 0 0.1f
M5673 t2115 nw115 vdd vdd pch w=2u l=180n
M5674 t2115 nw652 vdd vdd pch w=2u l=180n
CT2118 t2118 0 0.1f
M5675 t2115 nw115 t2118 0 nch w=1u l=180n
M5676 t2118 nw652 0 0 nch w=1u l=180n
M5677 t2116 nw115 vdd vdd pch w=2u l=180n
M5678 t2116 t2115 vdd vdd pch w=2u l=180n
CT2119 t2119 0 0.1f
M5679 t2116 nw115 t2119 0 nch w=1u l=180n
M5680 t2119 t2115 0 0 nch w=1u l=180n
M5681 t2117 nw652 vdd vdd pch w=2u l=180n
M5682 t2117 t2115 vdd vdd pch w=2u l=180n
CT2120 t2120 0 0.1f
M5683 t2117 nw652 t2120 0 nch w=1u l=180n
M5684 t2120 t2115 0 0 nch w=1u l=180n
M5685 nw723 t2116 vdd vdd pch w=2u l=180n
M5686 nw723 t2117 vdd vdd pch w=2u l=180n
CT2121 t2121 0 0.1f
M5687 nw723 t2116 t2121 0 nch w=1u l=180n
M5688 t2121 t2117 0 0 nch w=1u l=180n
Cnw723 nw723 0 2f
CT2122 t2122 0 0.1f
CT2123 t2123 0 0.1f
CT2124 t2124 0 0.1f
M5689 t2122 nw723 vdd vdd pch w=2u l=180n
M5690 t2122 nw722 vdd vdd pch w=2u l=180n
CT2125 t2125 0 0.1f
M5691 t2122 nw723 t2125 0 nch w=1u l=180n
M5692 t2125 nw722 0 0 nch w=1u l=180n
M5693 t2123 nw723 vdd vdd pch w=2u l=180n
M5694 t2123 t2122 vdd vdd pch w=2u l=180n
CT2126 t2126 0 0.1f
M5695 t2123 nw723 t2126 0 nch w=1u l=180n
M5696 t2126 t2122 0 0 nch w=1u l=180n
M5697 t2124 nw722 vdd vdd pch w=2u l=180n
M5698 t2124 t2122 vdd vdd pch w=2u l=180n
CT2127 t2127 0 0.1f
M5699 t2124 nw722 t2127 0 nch w=1u l=180n
M5700 t2127 t2122 0 0 nch w=1u l=180n
M5701 nw724 t2123 vdd vdd pch w=2u l=180n
M5702 nw724 t2124 vdd vdd pch w=2u l=180n
CT2128 t2128 0 0.1f
M5703 nw724 t2123 t2128 0 nch w=1u l=180n
M5704 t2128 t2124 0 0 nch w=1u l=180n
Cnw724 nw724 0 2f
M5705 nw725 nw115 vdd vdd pch w=2u l=180n
M5706 nw725 nw652 vdd vdd pch w=2u l=180n
CT2129 t2129 0 0.1f
M5707 nw725 nw115 t2129 0 nch w=1u l=180n
M5708 t2129 nw652 0 0 nch w=1u l=180n
Cnw725 nw725 0 2f
M5709 nw726 nw723 vdd vdd pch w=2u l=180n
M5710 nw726 nw722 vdd vdd pch w=2u l=180n
CT2130 t2130 0 0.1f
M5711 nw726 nw723 t2130 0 nch w=1u l=180n
M5712 t2130 nw722 0 0 nch w=1u l=180n
Cnw726 nw726 0 2f
M5713 nw727 nw725 vdd vdd pch w=2u l=180n
M5714 nw727 nw726 vdd vdd pch w=2u l=180n
CT2131 t2131 0 0.1f
M5715 nw727 nw725 t2131 0 nch w=1u l=180n
M5716 t2131 nw726 0 0 nch w=1u l=180n
Cnw727 nw727 0 2f
CT2132 t2132 0 0.1f
CT2133 t2133 0 0.1f
CT2134 t2134 0 0.1f
M5717 t2132 nw116 vdd vdd pch w=2u l=180n
M5718 t2132 nw657 vdd vdd pch w=2u l=180n
CT2135 t2135 0 0.1f
M5719 t2132 nw116 t2135 0 nch w=1u l=180n
M5720 t2135 nw657 0 0 nch w=1u l=180n
M5721 t2133 nw116 vdd vdd pch w=2u l=180n
M5722 t2133 t2132 vdd vdd pch w=2u l=180n
CT2136 t2136 0 0.1f
M5723 t2133 nw116 t2136 0 nch w=1u l=180n
M5724 t2136 t2132 0 0 nch w=1u l=180n
M5725 t2134 nw657 vdd vdd pch w=2u l=180n
M5726 t2134 t2132 vdd vdd pch w=2u l=180n
CT2137 t2137 0 0.1f
M5727 t2134 nw657 t2137 0 nch w=1u l=180n
M5728 t2137 t2132 0 0 nch w=1u l=180n
M5729 nw728 t2133 vdd vdd pch w=2u l=180n
M5730 nw728 t2134 vdd vdd pch w=2u l=180n
CT2138 t2138 0 0.1f
M5731 nw728 t2133 t2138 0 nch w=1u l=180n
M5732 t2138 t2134 0 0 nch w=1u l=180n
Cnw728 nw728 0 2f
CT2139 t2139 0 0.1f
CT2140 t2140 0 0.1f
CT2141 t2141 0 0.1f
M5733 t2139 nw728 vdd vdd pch w=2u l=180n
M5734 t2139 nw727 vdd vdd pch w=2u l=180n
CT2142 t2142 0 0.1f
M5735 t2139 nw728 t2142 0 nch w=1u l=180n
M5736 t2142 nw727 0 0 nch w=1u l=180n
M5737 t2140 nw728 vdd vdd pch w=2u l=180n
M5738 t2140 t2139 vdd vdd pch w=2u l=180n
CT2143 t2143 0 0.1f
M5739 t2140 nw728 t2143 0 nch w=1u l=180n
M5740 t2143 t2139 0 0 nch w=1u l=180n
M5741 t2141 nw727 vdd vdd pch w=2u l=180n
M5742 t2141 t2139 vdd vdd pch w=2u l=180n
CT2144 t2144 0 0.1f
M5743 t2141 nw727 t2144 0 nch w=1u l=180n
M5744 t2144 t2139 0 0 nch w=1u l=180n
M5745 nw729 t2140 vdd vdd pch w=2u l=180n
M5746 nw729 t2141 vdd vdd pch w=2u l=180n
CT2145 t2145 0 0.1f
M5747 nw729 t2140 t2145 0 nch w=1u l=180n
M5748 t2145 t2141 0 0 nch w=1u l=180n
Cnw729 nw729 0 2f
M5749 nw730 nw116 vdd vdd pch w=2u l=180n
M5750 nw730 nw657 vdd vdd pch w=2u l=180n
CT2146 t2146 0 0.1f
M5751 nw730 nw116 t2146 0 nch w=1u l=180n
M5752 t2146 nw657 0 0 nch w=1u l=180n
Cnw730 nw730 0 2f
M5753 nw731 nw728 vdd vdd pch w=2u l=180n
M5754 nw731 nw727 vdd vdd pch w=2u l=180n
CT2147 t2147 0 0.1f
M5755 nw731 nw728 t2147 0 nch w=1u l=180n
M5756 t2147 nw727 0 0 nch w=1u l=180n
Cnw731 nw731 0 2f
M5757 nw732 nw730 vdd vdd pch w=2u l=180n
M5758 nw732 nw731 vdd vdd pch w=2u l=180n
CT2148 t2148 0 0.1f
M5759 nw732 nw730 t2148 0 nch w=1u l=180n
M5760 t2148 nw731 0 0 nch w=1u l=180n
Cnw732 nw732 0 2f
CT2149 t2149 0 0.1f
CT2150 t2150 0 0.1f
CT2151 t2151 0 0.1f
M5761 t2149 nw117 vdd vdd pch w=2u l=180n
M5762 t2149 nw662 vdd vdd pch w=2u l=180n
CT2152 t2152 0 0.1f
M5763 t2149 nw117 t2152 0 nch w=1u l=180n
M5764 t2152 nw662 0 0 nch w=1u l=180n
M5765 t2150 nw117 vdd vdd pch w=2u l=180n
M5766 t2150 t2149 vdd vdd pch w=2u l=180n
CT2153 t2153 0 0.1f
M5767 t2150 nw117 t2153 0 nch w=1u l=180n
M5768 t2153 t2149 0 0 nch w=1u l=180n
M5769 t2151 nw662 vdd vdd pch w=2u l=180n
M5770 t2151 t2149 vdd vdd pch w=2u l=180n
CT2154 t2154 0 0.1f
M5771 t2151 nw662 t2154 0 nch w=1u l=180n
M5772 t2154 t2149 0 0 nch w=1u l=180n
M5773 nw733 t2150 vdd vdd pch w=2u l=180n
M5774 nw733 t2151 vdd vdd pch w=2u l=180n
CT2155 t2155 0 0.1f
M5775 nw733 t2150 t2155 0 nch w=1u l=180n
M5776 t2155 t2151 0 0 nch w=1u l=180n
Cnw733 nw733 0 2f
CT2156 t2156 0 0.1f
CT2157 t2157 0 0.1f
CT2158 t2158 0 0.1f
M5777 t2156 nw733 vdd vdd pch w=2u l=180n
M5778 t2156 nw732 vdd vdd pch w=2u l=180n
CT2159 t2159 0 0.1f
M5779 t2156 nw733 t2159 0 nch w=1u l=180n
M5780 t2159 nw732 0 0 nch w=1u l=180n
M5781 t2157 nw733 vdd vdd pch w=2u l=180n
M5782 t2157 t2156 vdd vdd pch w=2u l=180n
CT2160 t2160 0 0.1f
M5783 t2157 nw733 t2160 0 nch w=1u l=180n
M5784 t2160 t2156 0 0 nch w=1u l=180n
M5785 t2158 nw732 vdd vdd pch w=2u l=180n
M5786 t2158 t2156 vdd vdd pch w=2u l=180n
CT2161 t2161 0 0.1f
M5787 t2158 nw732 t2161 0 nch w=1u l=180n
M5788 t2161 t2156 0 0 nch w=1u l=180n
M5789 nw734 t2157 vdd vdd pch w=2u l=180n
M5790 nw734 t2158 vdd vdd pch w=2u l=180n
CT2162 t2162 0 0.1f
M5791 nw734 t2157 t2162 0 nch w=1u l=180n
M5792 t2162 t2158 0 0 nch w=1u l=180n
Cnw734 nw734 0 2f
M5793 nw735 nw117 vdd vdd pch w=2u l=180n
M5794 nw735 nw662 vdd vdd pch w=2u l=180n
CT2163 t2163 0 0.1f
M5795 nw735 nw117 t2163 0 nch w=1u l=180n
M5796 t2163 nw662 0 0 nch w=1u l=180n
Cnw735 nw735 0 2f
M5797 nw736 nw733 vdd vdd pch w=2u l=180n
M5798 nw736 nw732 vdd vdd pch w=2u l=180n
CT2164 t2164 0 0.1f
M5799 nw736 nw733 t2164 0 nch w=1u l=180n
M5800 t2164 nw732 0 0 nch w=1u l=180n
Cnw736 nw736 0 2f
M5801 nw737 nw735 vdd vdd pch w=2u l=180n
M5802 nw737 nw736 vdd vdd pch w=2u l=180n
CT2165 t2165 0 0.1f
M5803 nw737 nw735 t2165 0 nch w=1u l=180n
M5804 t2165 nw736 0 0 nch w=1u l=180n
Cnw737 nw737 0 2f
CT2166 t2166 0 0.1f
CT2167 t2167 0 0.1f
CT2168 t2168 0 0.1f
M5805 t2166 nw118 vdd vdd pch w=2u l=180n
M5806 t2166 nw667 vdd vdd pch w=2u l=180n
CT2169 t2169 0 0.1f
M5807 t2166 nw118 t2169 0 nch w=1u l=180n
M5808 t2169 nw667 0 0 nch w=1u l=180n
M5809 t2167 nw118 vdd vdd pch w=2u l=180n
M5810 t2167 t2166 vdd vdd pch w=2u l=180n
CT2170 t2170 0 0.1f
M5811 t2167 nw118 t2170 0 nch w=1u l=180n
M5812 t2170 t2166 0 0 nch w=1u l=180n
M5813 t2168 nw667 vdd vdd pch w=2u l=180n
M5814 t2168 t2166 vdd vdd pch w=2u l=180n
CT2171 t2171 0 0.1f
M5815 t2168 nw667 t2171 0 nch w=1u l=180n
M5816 t2171 t2166 0 0 nch w=1u l=180n
M5817 nw738 t2167 vdd vdd pch w=2u l=180n
M5818 nw738 t2168 vdd vdd pch w=2u l=180n
CT2172 t2172 0 0.1f
M5819 nw738 t2167 t2172 0 nch w=1u l=180n
M5820 t2172 t2168 0 0 nch w=1u l=180n
Cnw738 nw738 0 2f
CT2173 t2173 0 0.1f
CT2174 t2174 0 0.1f
CT2175 t2175 0 0.1f
M5821 t2173 nw738 vdd vdd pch w=2u l=180n
M5822 t2173 nw737 vdd vdd pch w=2u l=180n
CT2176 t2176 0 0.1f
M5823 t2173 nw738 t2176 0 nch w=1u l=180n
M5824 t2176 nw737 0 0 nch w=1u l=180n
M5825 t2174 nw738 vdd vdd pch w=2u l=180n
M5826 t2174 t2173 vdd vdd pch w=2u l=180n
CT2177 t2177 0 0.1f
M5827 t2174 nw738 t2177 0 nch w=1u l=180n
M5828 t2177 t2173 0 0 nch w=1u l=180n
M5829 t2175 nw737 vdd vdd pch w=2u l=180n
M5830 t2175 t2173 vdd vdd pch w=2u l=180n
CT2178 t2178 0 0.1f
M5831 t2175 nw737 t2178 0 nch w=1u l=180n
M5832 t2178 t2173 0 0 nch w=1u l=180n
M5833 nw739 t2174 vdd vdd pch w=2u l=180n
M5834 nw739 t2175 vdd vdd pch w=2u l=180n
CT2179 t2179 0 0.1f
M5835 nw739 t2174 t2179 0 nch w=1u l=180n
M5836 t2179 t2175 0 0 nch w=1u l=180n
Cnw739 nw739 0 2f
M5837 nw740 nw118 vdd vdd pch w=2u l=180n
M5838 nw740 nw667 vdd vdd pch w=2u l=180n
CT2180 t2180 0 0.1f
M5839 nw740 nw118 t2180 0 nch w=1u l=180n
M5840 t2180 nw667 0 0 nch w=1u l=180n
Cnw740 nw740 0 2f
M5841 nw741 nw738 vdd vdd pch w=2u l=180n
M5842 nw741 nw737 vdd vdd pch w=2u l=180n
CT2181 t2181 0 0.1f
M5843 nw741 nw738 t2181 0 nch w=1u l=180n
M5844 t2181 nw737 0 0 nch w=1u l=180n
Cnw741 nw741 0 2f
M5845 nw742 nw740 vdd vdd pch w=2u l=180n
M5846 nw742 nw741 vdd vdd pch w=2u l=180n
CT2182 t2182 0 0.1f
M5847 nw742 nw740 t2182 0 nch w=1u l=180n
M5848 t2182 nw741 0 0 nch w=1u l=180n
Cnw742 nw742 0 2f
CT2183 t2183 0 0.1f
CT2184 t2184 0 0.1f
CT2185 t2185 0 0.1f
M5849 t2183 nw119 vdd vdd pch w=2u l=180n
M5850 t2183 nw672 vdd vdd pch w=2u l=180n
CT2186 t2186 0 0.1f
M5851 t2183 nw119 t2186 0 nch w=1u l=180n
M5852 t2186 nw672 0 0 nch w=1u l=180n
M5853 t2184 nw119 vdd vdd pch w=2u l=180n
M5854 t2184 t2183 vdd vdd pch w=2u l=180n
CT2187 t2187 0 0.1f
M5855 t2184 nw119 t2187 0 nch w=1u l=180n
M5856 t2187 t2183 0 0 nch w=1u l=180n
M5857 t2185 nw672 vdd vdd pch w=2u l=180n
M5858 t2185 t2183 vdd vdd pch w=2u l=180n
CT2188 t2188 0 0.1f
M5859 t2185 nw672 t2188 0 nch w=1u l=180n
M5860 t2188 t2183 0 0 nch w=1u l=180n
M5861 nw743 t2184 vdd vdd pch w=2u l=180n
M5862 nw743 t2185 vdd vdd pch w=2u l=180n
CT2189 t2189 0 0.1f
M5863 nw743 t2184 t2189 0 nch w=1u l=180n
M5864 t2189 t2185 0 0 nch w=1u l=180n
Cnw743 nw743 0 2f
CT2190 t2190 0 0.1f
CT2191 t2191 0 0.1f
CT2192 t2192 0 0.1f
M5865 t2190 nw743 vdd vdd pch w=2u l=180n
M5866 t2190 nw742 vdd vdd pch w=2u l=180n
CT2193 t2193 0 0.1f
M5867 t2190 nw743 t2193 0 nch w=1u l=180n
M5868 t2193 nw742 0 0 nch w=1u l=180n
M5869 t2191 nw743 vdd vdd pch w=2u l=180n
M5870 t2191 t2190 vdd vdd pch w=2u l=180n
CT2194 t2194 0 0.1f
M5871 t2191 nw743 t2194 0 nch w=1u l=180n
M5872 t2194 t2190 0 0 nch w=1u l=180n
M5873 t2192 nw742 vdd vdd pch w=2u l=180n
M5874 t2192 t2190 vdd vdd pch w=2u l=180n
CT2195 t2195 0 0.1f
M5875 t2192 nw742 t2195 0 nch w=1u l=180n
M5876 t2195 t2190 0 0 nch w=1u l=180n
M5877 nw744 t2191 vdd vdd pch w=2u l=180n
M5878 nw744 t2192 vdd vdd pch w=2u l=180n
CT2196 t2196 0 0.1f
M5879 nw744 t2191 t2196 0 nch w=1u l=180n
M5880 t2196 t2192 0 0 nch w=1u l=180n
Cnw744 nw744 0 2f
M5881 nw745 nw119 vdd vdd pch w=2u l=180n
M5882 nw745 nw672 vdd vdd pch w=2u l=180n
CT2197 t2197 0 0.1f
M5883 nw745 nw119 t2197 0 nch w=1u l=180n
M5884 t2197 nw672 0 0 nch w=1u l=180n
Cnw745 nw745 0 2f
M5885 nw746 nw743 vdd vdd pch w=2u l=180n
M5886 nw746 nw742 vdd vdd pch w=2u l=180n
CT2198 t2198 0 0.1f
M5887 nw746 nw743 t2198 0 nch w=1u l=180n
M5888 t2198 nw742 0 0 nch w=1u l=180n
Cnw746 nw746 0 2f
M5889 nw747 nw745 vdd vdd pch w=2u l=180n
M5890 nw747 nw746 vdd vdd pch w=2u l=180n
CT2199 t2199 0 0.1f
M5891 nw747 nw745 t2199 0 nch w=1u l=180n
M5892 t2199 nw746 0 0 nch w=1u l=180n
Cnw747 nw747 0 2f
CT2200 t2200 0 0.1f
CT2201 t2201 0 0.1f
CT2202 t2202 0 0.1f
M5893 t2200 nw120 vdd vdd pch w=2u l=180n
M5894 t2200 nw677 vdd vdd pch w=2u l=180n
CT2203 t2203 0 0.1f
M5895 t2200 nw120 t2203 0 nch w=1u l=180n
M5896 t2203 nw677 0 0 nch w=1u l=180n
M5897 t2201 nw120 vdd vdd pch w=2u l=180n
M5898 t2201 t2200 vdd vdd pch w=2u l=180n
CT2204 t2204 0 0.1f
M5899 t2201 nw120 t2204 0 nch w=1u l=180n
M5900 t2204 t2200 0 0 nch w=1u l=180n
M5901 t2202 nw677 vdd vdd pch w=2u l=180n
M5902 t2202 t2200 vdd vdd pch w=2u l=180n
CT2205 t2205 0 0.1f
M5903 t2202 nw677 t2205 0 nch w=1u l=180n
M5904 t2205 t2200 0 0 nch w=1u l=180n
M5905 nw748 t2201 vdd vdd pch w=2u l=180n
M5906 nw748 t2202 vdd vdd pch w=2u l=180n
CT2206 t2206 0 0.1f
M5907 nw748 t2201 t2206 0 nch w=1u l=180n
M5908 t2206 t2202 0 0 nch w=1u l=180n
Cnw748 nw748 0 2f
CT2207 t2207 0 0.1f
CT2208 t2208 0 0.1f
CT2209 t2209 0 0.1f
M5909 t2207 nw748 vdd vdd pch w=2u l=180n
M5910 t2207 nw747 vdd vdd pch w=2u l=180n
CT2210 t2210 0 0.1f
M5911 t2207 nw748 t2210 0 nch w=1u l=180n
M5912 t2210 nw747 0 0 nch w=1u l=180n
M5913 t2208 nw748 vdd vdd pch w=2u l=180n
M5914 t2208 t2207 vdd vdd pch w=2u l=180n
CT2211 t2211 0 0.1f
M5915 t2208 nw748 t2211 0 nch w=1u l=180n
M5916 t2211 t2207 0 0 nch w=1u l=180n
M5917 t2209 nw747 vdd vdd pch w=2u l=180n
M5918 t2209 t2207 vdd vdd pch w=2u l=180n
CT2212 t2212 0 0.1f
M5919 t2209 nw747 t2212 0 nch w=1u l=180n
M5920 t2212 t2207 0 0 nch w=1u l=180n
M5921 nw749 t2208 vdd vdd pch w=2u l=180n
M5922 nw749 t2209 vdd vdd pch w=2u l=180n
CT2213 t2213 0 0.1f
M5923 nw749 t2208 t2213 0 nch w=1u l=180n
M5924 t2213 t2209 0 0 nch w=1u l=180n
Cnw749 nw749 0 2f
M5925 nw750 nw120 vdd vdd pch w=2u l=180n
M5926 nw750 nw677 vdd vdd pch w=2u l=180n
CT2214 t2214 0 0.1f
M5927 nw750 nw120 t2214 0 nch w=1u l=180n
M5928 t2214 nw677 0 0 nch w=1u l=180n
Cnw750 nw750 0 2f
M5929 nw751 nw748 vdd vdd pch w=2u l=180n
M5930 nw751 nw747 vdd vdd pch w=2u l=180n
CT2215 t2215 0 0.1f
M5931 nw751 nw748 t2215 0 nch w=1u l=180n
M5932 t2215 nw747 0 0 nch w=1u l=180n
Cnw751 nw751 0 2f
M5933 nw752 nw750 vdd vdd pch w=2u l=180n
M5934 nw752 nw751 vdd vdd pch w=2u l=180n
CT2216 t2216 0 0.1f
M5935 nw752 nw750 t2216 0 nch w=1u l=180n
M5936 t2216 nw751 0 0 nch w=1u l=180n
Cnw752 nw752 0 2f
CT2217 t2217 0 0.1f
CT2218 t2218 0 0.1f
CT2219 t2219 0 0.1f
M5937 t2217 nw121 vdd vdd pch w=2u l=180n
M5938 t2217 nw682 vdd vdd pch w=2u l=180n
CT2220 t2220 0 0.1f
M5939 t2217 nw121 t2220 0 nch w=1u l=180n
M5940 t2220 nw682 0 0 nch w=1u l=180n
M5941 t2218 nw121 vdd vdd pch w=2u l=180n
M5942 t2218 t2217 vdd vdd pch w=2u l=180n
CT2221 t2221 0 0.1f
M5943 t2218 nw121 t2221 0 nch w=1u l=180n
M5944 t2221 t2217 0 0 nch w=1u l=180n
M5945 t2219 nw682 vdd vdd pch w=2u l=180n
M5946 t2219 t2217 vdd vdd pch w=2u l=180n
CT2222 t2222 0 0.1f
M5947 t2219 nw682 t2222 0 nch w=1u l=180n
M5948 t2222 t2217 0 0 nch w=1u l=180n
M5949 nw753 t2218 vdd vdd pch w=2u l=180n
M5950 nw753 t2219 vdd vdd pch w=2u l=180n
CT2223 t2223 0 0.1f
M5951 nw753 t2218 t2223 0 nch w=1u l=180n
M5952 t2223 t2219 0 0 nch w=1u l=180n
Cnw753 nw753 0 2f
CT2224 t2224 0 0.1f
CT2225 t2225 0 0.1f
CT2226 t2226 0 0.1f
M5953 t2224 nw753 vdd vdd pch w=2u l=180n
M5954 t2224 nw752 vdd vdd pch w=2u l=180n
CT2227 t2227 0 0.1f
M5955 t2224 nw753 t2227 0 nch w=1u l=180n
M5956 t2227 nw752 0 0 nch w=1u l=180n
M5957 t2225 nw753 vdd vdd pch w=2u l=180n
M5958 t2225 t2224 vdd vdd pch w=2u l=180n
CT2228 t2228 0 0.1f
M5959 t2225 nw753 t2228 0 nch w=1u l=180n
M5960 t2228 t2224 0 0 nch w=1u l=180n
M5961 t2226 nw752 vdd vdd pch w=2u l=180n
M5962 t2226 t2224 vdd vdd pch w=2u l=180n
CT2229 t2229 0 0.1f
M5963 t2226 nw752 t2229 0 nch w=1u l=180n
M5964 t2229 t2224 0 0 nch w=1u l=180n
M5965 nw754 t2225 vdd vdd pch w=2u l=180n
M5966 nw754 t2226 vdd vdd pch w=2u l=180n
CT2230 t2230 0 0.1f
M5967 nw754 t2225 t2230 0 nch w=1u l=180n
M5968 t2230 t2226 0 0 nch w=1u l=180n
Cnw754 nw754 0 2f
M5969 nw755 nw121 vdd vdd pch w=2u l=180n
M5970 nw755 nw682 vdd vdd pch w=2u l=180n
CT2231 t2231 0 0.1f
M5971 nw755 nw121 t2231 0 nch w=1u l=180n
M5972 t2231 nw682 0 0 nch w=1u l=180n
Cnw755 nw755 0 2f
M5973 nw756 nw753 vdd vdd pch w=2u l=180n
M5974 nw756 nw752 vdd vdd pch w=2u l=180n
CT2232 t2232 0 0.1f
M5975 nw756 nw753 t2232 0 nch w=1u l=180n
M5976 t2232 nw752 0 0 nch w=1u l=180n
Cnw756 nw756 0 2f
M5977 nw757 nw755 vdd vdd pch w=2u l=180n
M5978 nw757 nw756 vdd vdd pch w=2u l=180n
CT2233 t2233 0 0.1f
M5979 nw757 nw755 t2233 0 nch w=1u l=180n
M5980 t2233 nw756 0 0 nch w=1u l=180n
Cnw757 nw757 0 2f
CT2234 t2234 0 0.1f
CT2235 t2235 0 0.1f
CT2236 t2236 0 0.1f
M5981 t2234 nw122 vdd vdd pch w=2u l=180n
M5982 t2234 nw687 vdd vdd pch w=2u l=180n
CT2237 t2237 0 0.1f
M5983 t2234 nw122 t2237 0 nch w=1u l=180n
M5984 t2237 nw687 0 0 nch w=1u l=180n
M5985 t2235 nw122 vdd vdd pch w=2u l=180n
M5986 t2235 t2234 vdd vdd pch w=2u l=180n
CT2238 t2238 0 0.1f
M5987 t2235 nw122 t2238 0 nch w=1u l=180n
M5988 t2238 t2234 0 0 nch w=1u l=180n
M5989 t2236 nw687 vdd vdd pch w=2u l=180n
M5990 t2236 t2234 vdd vdd pch w=2u l=180n
CT2239 t2239 0 0.1f
M5991 t2236 nw687 t2239 0 nch w=1u l=180n
M5992 t2239 t2234 0 0 nch w=1u l=180n
M5993 nw758 t2235 vdd vdd pch w=2u l=180n
M5994 nw758 t2236 vdd vdd pch w=2u l=180n
CT2240 t2240 0 0.1f
M5995 nw758 t2235 t2240 0 nch w=1u l=180n
M5996 t2240 t2236 0 0 nch w=1u l=180n
Cnw758 nw758 0 2f
CT2241 t2241 0 0.1f
CT2242 t2242 0 0.1f
CT2243 t2243 0 0.1f
M5997 t2241 nw758 vdd vdd pch w=2u l=180n
M5998 t2241 nw757 vdd vdd pch w=2u l=180n
CT2244 t2244 0 0.1f
M5999 t2241 nw758 t2244 0 nch w=1u l=180n
M6000 t2244 nw757 0 0 nch w=1u l=180n
M6001 t2242 nw758 vdd vdd pch w=2u l=180n
M6002 t2242 t2241 vdd vdd pch w=2u l=180n
CT2245 t2245 0 0.1f
M6003 t2242 nw758 t2245 0 nch w=1u l=180n
M6004 t2245 t2241 0 0 nch w=1u l=180n
M6005 t2243 nw757 vdd vdd pch w=2u l=180n
M6006 t2243 t2241 vdd vdd pch w=2u l=180n
CT2246 t2246 0 0.1f
M6007 t2243 nw757 t2246 0 nch w=1u l=180n
M6008 t2246 t2241 0 0 nch w=1u l=180n
M6009 nw759 t2242 vdd vdd pch w=2u l=180n
M6010 nw759 t2243 vdd vdd pch w=2u l=180n
CT2247 t2247 0 0.1f
M6011 nw759 t2242 t2247 0 nch w=1u l=180n
M6012 t2247 t2243 0 0 nch w=1u l=180n
Cnw759 nw759 0 2f
M6013 nw760 nw122 vdd vdd pch w=2u l=180n
M6014 nw760 nw687 vdd vdd pch w=2u l=180n
CT2248 t2248 0 0.1f
M6015 nw760 nw122 t2248 0 nch w=1u l=180n
M6016 t2248 nw687 0 0 nch w=1u l=180n
Cnw760 nw760 0 2f
M6017 nw761 nw758 vdd vdd pch w=2u l=180n
M6018 nw761 nw757 vdd vdd pch w=2u l=180n
CT2249 t2249 0 0.1f
M6019 nw761 nw758 t2249 0 nch w=1u l=180n
M6020 t2249 nw757 0 0 nch w=1u l=180n
Cnw761 nw761 0 2f
M6021 nw762 nw760 vdd vdd pch w=2u l=180n
M6022 nw762 nw761 vdd vdd pch w=2u l=180n
CT2250 t2250 0 0.1f
M6023 nw762 nw760 t2250 0 nch w=1u l=180n
M6024 t2250 nw761 0 0 nch w=1u l=180n
Cnw762 nw762 0 2f
CT2251 t2251 0 0.1f
CT2252 t2252 0 0.1f
CT2253 t2253 0 0.1f
M6025 t2251 nw123 vdd vdd pch w=2u l=180n
M6026 t2251 nw692 vdd vdd pch w=2u l=180n
CT2254 t2254 0 0.1f
M6027 t2251 nw123 t2254 0 nch w=1u l=180n
M6028 t2254 nw692 0 0 nch w=1u l=180n
M6029 t2252 nw123 vdd vdd pch w=2u l=180n
M6030 t2252 t2251 vdd vdd pch w=2u l=180n
CT2255 t2255 0 0.1f
M6031 t2252 nw123 t2255 0 nch w=1u l=180n
M6032 t2255 t2251 0 0 nch w=1u l=180n
M6033 t2253 nw692 vdd vdd pch w=2u l=180n
M6034 t2253 t2251 vdd vdd pch w=2u l=180n
CT2256 t2256 0 0.1f
M6035 t2253 nw692 t2256 0 nch w=1u l=180n
M6036 t2256 t2251 0 0 nch w=1u l=180n
M6037 nw763 t2252 vdd vdd pch w=2u l=180n
M6038 nw763 t2253 vdd vdd pch w=2u l=180n
CT2257 t2257 0 0.1f
M6039 nw763 t2252 t2257 0 nch w=1u l=180n
M6040 t2257 t2253 0 0 nch w=1u l=180n
Cnw763 nw763 0 2f
CT2258 t2258 0 0.1f
CT2259 t2259 0 0.1f
CT2260 t2260 0 0.1f
M6041 t2258 nw763 vdd vdd pch w=2u l=180n
M6042 t2258 nw762 vdd vdd pch w=2u l=180n
CT2261 t2261 0 0.1f
M6043 t2258 nw763 t2261 0 nch w=1u l=180n
M6044 t2261 nw762 0 0 nch w=1u l=180n
M6045 t2259 nw763 vdd vdd pch w=2u l=180n
M6046 t2259 t2258 vdd vdd pch w=2u l=180n
CT2262 t2262 0 0.1f
M6047 t2259 nw763 t2262 0 nch w=1u l=180n
M6048 t2262 t2258 0 0 nch w=1u l=180n
M6049 t2260 nw762 vdd vdd pch w=2u l=180n
M6050 t2260 t2258 vdd vdd pch w=2u l=180n
CT2263 t2263 0 0.1f
M6051 t2260 nw762 t2263 0 nch w=1u l=180n
M6052 t2263 t2258 0 0 nch w=1u l=180n
M6053 nw764 t2259 vdd vdd pch w=2u l=180n
M6054 nw764 t2260 vdd vdd pch w=2u l=180n
CT2264 t2264 0 0.1f
M6055 nw764 t2259 t2264 0 nch w=1u l=180n
M6056 t2264 t2260 0 0 nch w=1u l=180n
Cnw764 nw764 0 2f
M6057 nw765 nw123 vdd vdd pch w=2u l=180n
M6058 nw765 nw692 vdd vdd pch w=2u l=180n
CT2265 t2265 0 0.1f
M6059 nw765 nw123 t2265 0 nch w=1u l=180n
M6060 t2265 nw692 0 0 nch w=1u l=180n
Cnw765 nw765 0 2f
M6061 nw766 nw763 vdd vdd pch w=2u l=180n
M6062 nw766 nw762 vdd vdd pch w=2u l=180n
CT2266 t2266 0 0.1f
M6063 nw766 nw763 t2266 0 nch w=1u l=180n
M6064 t2266 nw762 0 0 nch w=1u l=180n
Cnw766 nw766 0 2f
M6065 nw767 nw765 vdd vdd pch w=2u l=180n
M6066 nw767 nw766 vdd vdd pch w=2u l=180n
CT2267 t2267 0 0.1f
M6067 nw767 nw765 t2267 0 nch w=1u l=180n
M6068 t2267 nw766 0 0 nch w=1u l=180n
Cnw767 nw767 0 2f
CT2268 t2268 0 0.1f
CT2269 t2269 0 0.1f
CT2270 t2270 0 0.1f
M6069 t2268 nw124 vdd vdd pch w=2u l=180n
M6070 t2268 nw697 vdd vdd pch w=2u l=180n
CT2271 t2271 0 0.1f
M6071 t2268 nw124 t2271 0 nch w=1u l=180n
M6072 t2271 nw697 0 0 nch w=1u l=180n
M6073 t2269 nw124 vdd vdd pch w=2u l=180n
M6074 t2269 t2268 vdd vdd pch w=2u l=180n
CT2272 t2272 0 0.1f
M6075 t2269 nw124 t2272 0 nch w=1u l=180n
M6076 t2272 t2268 0 0 nch w=1u l=180n
M6077 t2270 nw697 vdd vdd pch w=2u l=180n
M6078 t2270 t2268 vdd vdd pch w=2u l=180n
CT2273 t2273 0 0.1f
M6079 t2270 nw697 t2273 0 nch w=1u l=180n
M6080 t2273 t2268 0 0 nch w=1u l=180n
M6081 nw768 t2269 vdd vdd pch w=2u l=180n
M6082 nw768 t2270 vdd vdd pch w=2u l=180n
CT2274 t2274 0 0.1f
M6083 nw768 t2269 t2274 0 nch w=1u l=180n
M6084 t2274 t2270 0 0 nch w=1u l=180n
Cnw768 nw768 0 2f
CT2275 t2275 0 0.1f
CT2276 t2276 0 0.1f
CT2277 t2277 0 0.1f
M6085 t2275 nw768 vdd vdd pch w=2u l=180n
M6086 t2275 nw767 vdd vdd pch w=2u l=180n
CT2278 t2278 0 0.1f
M6087 t2275 nw768 t2278 0 nch w=1u l=180n
M6088 t2278 nw767 0 0 nch w=1u l=180n
M6089 t2276 nw768 vdd vdd pch w=2u l=180n
M6090 t2276 t2275 vdd vdd pch w=2u l=180n
CT2279 t2279 0 0.1f
M6091 t2276 nw768 t2279 0 nch w=1u l=180n
M6092 t2279 t2275 0 0 nch w=1u l=180n
M6093 t2277 nw767 vdd vdd pch w=2u l=180n
M6094 t2277 t2275 vdd vdd pch w=2u l=180n
CT2280 t2280 0 0.1f
M6095 t2277 nw767 t2280 0 nch w=1u l=180n
M6096 t2280 t2275 0 0 nch w=1u l=180n
M6097 nw769 t2276 vdd vdd pch w=2u l=180n
M6098 nw769 t2277 vdd vdd pch w=2u l=180n
CT2281 t2281 0 0.1f
M6099 nw769 t2276 t2281 0 nch w=1u l=180n
M6100 t2281 t2277 0 0 nch w=1u l=180n
Cnw769 nw769 0 2f
M6101 nw770 nw124 vdd vdd pch w=2u l=180n
M6102 nw770 nw697 vdd vdd pch w=2u l=180n
CT2282 t2282 0 0.1f
M6103 nw770 nw124 t2282 0 nch w=1u l=180n
M6104 t2282 nw697 0 0 nch w=1u l=180n
Cnw770 nw770 0 2f
M6105 nw771 nw768 vdd vdd pch w=2u l=180n
M6106 nw771 nw767 vdd vdd pch w=2u l=180n
CT2283 t2283 0 0.1f
M6107 nw771 nw768 t2283 0 nch w=1u l=180n
M6108 t2283 nw767 0 0 nch w=1u l=180n
Cnw771 nw771 0 2f
M6109 nw772 nw770 vdd vdd pch w=2u l=180n
M6110 nw772 nw771 vdd vdd pch w=2u l=180n
CT2284 t2284 0 0.1f
M6111 nw772 nw770 t2284 0 nch w=1u l=180n
M6112 t2284 nw771 0 0 nch w=1u l=180n
Cnw772 nw772 0 2f
CT2285 t2285 0 0.1f
CT2286 t2286 0 0.1f
CT2287 t2287 0 0.1f
M6113 t2285 nw125 vdd vdd pch w=2u l=180n
M6114 t2285 nw702 vdd vdd pch w=2u l=180n
CT2288 t2288 0 0.1f
M6115 t2285 nw125 t2288 0 nch w=1u l=180n
M6116 t2288 nw702 0 0 nch w=1u l=180n
M6117 t2286 nw125 vdd vdd pch w=2u l=180n
M6118 t2286 t2285 vdd vdd pch w=2u l=180n
CT2289 t2289 0 0.1f
M6119 t2286 nw125 t2289 0 nch w=1u l=180n
M6120 t2289 t2285 0 0 nch w=1u l=180n
M6121 t2287 nw702 vdd vdd pch w=2u l=180n
M6122 t2287 t2285 vdd vdd pch w=2u l=180n
CT2290 t2290 0 0.1f
M6123 t2287 nw702 t2290 0 nch w=1u l=180n
M6124 t2290 t2285 0 0 nch w=1u l=180n
M6125 nw773 t2286 vdd vdd pch w=2u l=180n
M6126 nw773 t2287 vdd vdd pch w=2u l=180n
CT2291 t2291 0 0.1f
M6127 nw773 t2286 t2291 0 nch w=1u l=180n
M6128 t2291 t2287 0 0 nch w=1u l=180n
Cnw773 nw773 0 2f
CT2292 t2292 0 0.1f
CT2293 t2293 0 0.1f
CT2294 t2294 0 0.1f
M6129 t2292 nw773 vdd vdd pch w=2u l=180n
M6130 t2292 nw772 vdd vdd pch w=2u l=180n
CT2295 t2295 0 0.1f
M6131 t2292 nw773 t2295 0 nch w=1u l=180n
M6132 t2295 nw772 0 0 nch w=1u l=180n
M6133 t2293 nw773 vdd vdd pch w=2u l=180n
M6134 t2293 t2292 vdd vdd pch w=2u l=180n
CT2296 t2296 0 0.1f
M6135 t2293 nw773 t2296 0 nch w=1u l=180n
M6136 t2296 t2292 0 0 nch w=1u l=180n
M6137 t2294 nw772 vdd vdd pch w=2u l=180n
M6138 t2294 t2292 vdd vdd pch w=2u l=180n
CT2297 t2297 0 0.1f
M6139 t2294 nw772 t2297 0 nch w=1u l=180n
M6140 t2297 t2292 0 0 nch w=1u l=180n
M6141 nw774 t2293 vdd vdd pch w=2u l=180n
M6142 nw774 t2294 vdd vdd pch w=2u l=180n
CT2298 t2298 0 0.1f
M6143 nw774 t2293 t2298 0 nch w=1u l=180n
M6144 t2298 t2294 0 0 nch w=1u l=180n
Cnw774 nw774 0 2f
M6145 nw775 nw125 vdd vdd pch w=2u l=180n
M6146 nw775 nw702 vdd vdd pch w=2u l=180n
CT2299 t2299 0 0.1f
M6147 nw775 nw125 t2299 0 nch w=1u l=180n
M6148 t2299 nw702 0 0 nch w=1u l=180n
Cnw775 nw775 0 2f
M6149 nw776 nw773 vdd vdd pch w=2u l=180n
M6150 nw776 nw772 vdd vdd pch w=2u l=180n
CT2300 t2300 0 0.1f
M6151 nw776 nw773 t2300 0 nch w=1u l=180n
M6152 t2300 nw772 0 0 nch w=1u l=180n
Cnw776 nw776 0 2f
M6153 nw777 nw775 vdd vdd pch w=2u l=180n
M6154 nw777 nw776 vdd vdd pch w=2u l=180n
CT2301 t2301 0 0.1f
M6155 nw777 nw775 t2301 0 nch w=1u l=180n
M6156 t2301 nw776 0 0 nch w=1u l=180n
Cnw777 nw777 0 2f
CT2302 t2302 0 0.1f
CT2303 t2303 0 0.1f
CT2304 t2304 0 0.1f
M6157 t2302 nw126 vdd vdd pch w=2u l=180n
M6158 t2302 nw707 vdd vdd pch w=2u l=180n
CT2305 t2305 0 0.1f
M6159 t2302 nw126 t2305 0 nch w=1u l=180n
M6160 t2305 nw707 0 0 nch w=1u l=180n
M6161 t2303 nw126 vdd vdd pch w=2u l=180n
M6162 t2303 t2302 vdd vdd pch w=2u l=180n
CT2306 t2306 0 0.1f
M6163 t2303 nw126 t2306 0 nch w=1u l=180n
M6164 t2306 t2302 0 0 nch w=1u l=180n
M6165 t2304 nw707 vdd vdd pch w=2u l=180n
M6166 t2304 t2302 vdd vdd pch w=2u l=180n
CT2307 t2307 0 0.1f
M6167 t2304 nw707 t2307 0 nch w=1u l=180n
M6168 t2307 t2302 0 0 nch w=1u l=180n
M6169 nw778 t2303 vdd vdd pch w=2u l=180n
M6170 nw778 t2304 vdd vdd pch w=2u l=180n
CT2308 t2308 0 0.1f
M6171 nw778 t2303 t2308 0 nch w=1u l=180n
M6172 t2308 t2304 0 0 nch w=1u l=180n
Cnw778 nw778 0 2f
CT2309 t2309 0 0.1f
CT2310 t2310 0 0.1f
CT2311 t2311 0 0.1f
M6173 t2309 nw778 vdd vdd pch w=2u l=180n
M6174 t2309 nw777 vdd vdd pch w=2u l=180n
CT2312 t2312 0 0.1f
M6175 t2309 nw778 t2312 0 nch w=1u l=180n
M6176 t2312 nw777 0 0 nch w=1u l=180n
M6177 t2310 nw778 vdd vdd pch w=2u l=180n
M6178 t2310 t2309 vdd vdd pch w=2u l=180n
CT2313 t2313 0 0.1f
M6179 t2310 nw778 t2313 0 nch w=1u l=180n
M6180 t2313 t2309 0 0 nch w=1u l=180n
M6181 t2311 nw777 vdd vdd pch w=2u l=180n
M6182 t2311 t2309 vdd vdd pch w=2u l=180n
CT2314 t2314 0 0.1f
M6183 t2311 nw777 t2314 0 nch w=1u l=180n
M6184 t2314 t2309 0 0 nch w=1u l=180n
M6185 nw779 t2310 vdd vdd pch w=2u l=180n
M6186 nw779 t2311 vdd vdd pch w=2u l=180n
CT2315 t2315 0 0.1f
M6187 nw779 t2310 t2315 0 nch w=1u l=180n
M6188 t2315 t2311 0 0 nch w=1u l=180n
Cnw779 nw779 0 2f
M6189 nw780 nw126 vdd vdd pch w=2u l=180n
M6190 nw780 nw707 vdd vdd pch w=2u l=180n
CT2316 t2316 0 0.1f
M6191 nw780 nw126 t2316 0 nch w=1u l=180n
M6192 t2316 nw707 0 0 nch w=1u l=180n
Cnw780 nw780 0 2f
M6193 nw781 nw778 vdd vdd pch w=2u l=180n
M6194 nw781 nw777 vdd vdd pch w=2u l=180n
CT2317 t2317 0 0.1f
M6195 nw781 nw778 t2317 0 nch w=1u l=180n
M6196 t2317 nw777 0 0 nch w=1u l=180n
Cnw781 nw781 0 2f
M6197 nw782 nw780 vdd vdd pch w=2u l=180n
M6198 nw782 nw781 vdd vdd pch w=2u l=180n
CT2318 t2318 0 0.1f
M6199 nw782 nw780 t2318 0 nch w=1u l=180n
M6200 t2318 nw781 0 0 nch w=1u l=180n
Cnw782 nw782 0 2f
CT2319 t2319 0 0.1f
CT2320 t2320 0 0.1f
CT2321 t2321 0 0.1f
M6201 t2319 nw127 vdd vdd pch w=2u l=180n
M6202 t2319 nw712 vdd vdd pch w=2u l=180n
CT2322 t2322 0 0.1f
M6203 t2319 nw127 t2322 0 nch w=1u l=180n
M6204 t2322 nw712 0 0 nch w=1u l=180n
M6205 t2320 nw127 vdd vdd pch w=2u l=180n
M6206 t2320 t2319 vdd vdd pch w=2u l=180n
CT2323 t2323 0 0.1f
M6207 t2320 nw127 t2323 0 nch w=1u l=180n
M6208 t2323 t2319 0 0 nch w=1u l=180n
M6209 t2321 nw712 vdd vdd pch w=2u l=180n
M6210 t2321 t2319 vdd vdd pch w=2u l=180n
CT2324 t2324 0 0.1f
M6211 t2321 nw712 t2324 0 nch w=1u l=180n
M6212 t2324 t2319 0 0 nch w=1u l=180n
M6213 nw783 t2320 vdd vdd pch w=2u l=180n
M6214 nw783 t2321 vdd vdd pch w=2u l=180n
CT2325 t2325 0 0.1f
M6215 nw783 t2320 t2325 0 nch w=1u l=180n
M6216 t2325 t2321 0 0 nch w=1u l=180n
Cnw783 nw783 0 2f
CT2326 t2326 0 0.1f
CT2327 t2327 0 0.1f
CT2328 t2328 0 0.1f
M6217 t2326 nw783 vdd vdd pch w=2u l=180n
M6218 t2326 nw782 vdd vdd pch w=2u l=180n
CT2329 t2329 0 0.1f
M6219 t2326 nw783 t2329 0 nch w=1u l=180n
M6220 t2329 nw782 0 0 nch w=1u l=180n
M6221 t2327 nw783 vdd vdd pch w=2u l=180n
M6222 t2327 t2326 vdd vdd pch w=2u l=180n
CT2330 t2330 0 0.1f
M6223 t2327 nw783 t2330 0 nch w=1u l=180n
M6224 t2330 t2326 0 0 nch w=1u l=180n
M6225 t2328 nw782 vdd vdd pch w=2u l=180n
M6226 t2328 t2326 vdd vdd pch w=2u l=180n
CT2331 t2331 0 0.1f
M6227 t2328 nw782 t2331 0 nch w=1u l=180n
M6228 t2331 t2326 0 0 nch w=1u l=180n
M6229 nw784 t2327 vdd vdd pch w=2u l=180n
M6230 nw784 t2328 vdd vdd pch w=2u l=180n
CT2332 t2332 0 0.1f
M6231 nw784 t2327 t2332 0 nch w=1u l=180n
M6232 t2332 t2328 0 0 nch w=1u l=180n
Cnw784 nw784 0 2f
M6233 nw785 nw127 vdd vdd pch w=2u l=180n
M6234 nw785 nw712 vdd vdd pch w=2u l=180n
CT2333 t2333 0 0.1f
M6235 nw785 nw127 t2333 0 nch w=1u l=180n
M6236 t2333 nw712 0 0 nch w=1u l=180n
Cnw785 nw785 0 2f
M6237 nw786 nw783 vdd vdd pch w=2u l=180n
M6238 nw786 nw782 vdd vdd pch w=2u l=180n
CT2334 t2334 0 0.1f
M6239 nw786 nw783 t2334 0 nch w=1u l=180n
M6240 t2334 nw782 0 0 nch w=1u l=180n
Cnw786 nw786 0 2f
M6241 nw787 nw785 vdd vdd pch w=2u l=180n
M6242 nw787 nw786 vdd vdd pch w=2u l=180n
CT2335 t2335 0 0.1f
M6243 nw787 nw785 t2335 0 nch w=1u l=180n
M6244 t2335 nw786 0 0 nch w=1u l=180n
Cnw787 nw787 0 2f
CT2336 t2336 0 0.1f
CT2337 t2337 0 0.1f
CT2338 t2338 0 0.1f
M6245 t2336 nw128 vdd vdd pch w=2u l=180n
M6246 t2336 nw715 vdd vdd pch w=2u l=180n
CT2339 t2339 0 0.1f
M6247 t2336 nw128 t2339 0 nch w=1u l=180n
M6248 t2339 nw715 0 0 nch w=1u l=180n
M6249 t2337 nw128 vdd vdd pch w=2u l=180n
M6250 t2337 t2336 vdd vdd pch w=2u l=180n
CT2340 t2340 0 0.1f
M6251 t2337 nw128 t2340 0 nch w=1u l=180n
M6252 t2340 t2336 0 0 nch w=1u l=180n
M6253 t2338 nw715 vdd vdd pch w=2u l=180n
M6254 t2338 t2336 vdd vdd pch w=2u l=180n
CT2341 t2341 0 0.1f
M6255 t2338 nw715 t2341 0 nch w=1u l=180n
M6256 t2341 t2336 0 0 nch w=1u l=180n
M6257 nw788 t2337 vdd vdd pch w=2u l=180n
M6258 nw788 t2338 vdd vdd pch w=2u l=180n
CT2342 t2342 0 0.1f
M6259 nw788 t2337 t2342 0 nch w=1u l=180n
M6260 t2342 t2338 0 0 nch w=1u l=180n
Cnw788 nw788 0 2f
CT2343 t2343 0 0.1f
CT2344 t2344 0 0.1f
CT2345 t2345 0 0.1f
M6261 t2343 nw788 vdd vdd pch w=2u l=180n
M6262 t2343 nw787 vdd vdd pch w=2u l=180n
CT2346 t2346 0 0.1f
M6263 t2343 nw788 t2346 0 nch w=1u l=180n
M6264 t2346 nw787 0 0 nch w=1u l=180n
M6265 t2344 nw788 vdd vdd pch w=2u l=180n
M6266 t2344 t2343 vdd vdd pch w=2u l=180n
CT2347 t2347 0 0.1f
M6267 t2344 nw788 t2347 0 nch w=1u l=180n
M6268 t2347 t2343 0 0 nch w=1u l=180n
M6269 t2345 nw787 vdd vdd pch w=2u l=180n
M6270 t2345 t2343 vdd vdd pch w=2u l=180n
CT2348 t2348 0 0.1f
M6271 t2345 nw787 t2348 0 nch w=1u l=180n
M6272 t2348 t2343 0 0 nch w=1u l=180n
M6273 nw789 t2344 vdd vdd pch w=2u l=180n
M6274 nw789 t2345 vdd vdd pch w=2u l=180n
CT2349 t2349 0 0.1f
M6275 nw789 t2344 t2349 0 nch w=1u l=180n
M6276 t2349 t2345 0 0 nch w=1u l=180n
Cnw789 nw789 0 2f
M6277 nw790 nw128 vdd vdd pch w=2u l=180n
M6278 nw790 nw715 vdd vdd pch w=2u l=180n
CT2350 t2350 0 0.1f
M6279 nw790 nw128 t2350 0 nch w=1u l=180n
M6280 t2350 nw715 0 0 nch w=1u l=180n
Cnw790 nw790 0 2f
M6281 nw791 nw788 vdd vdd pch w=2u l=180n
M6282 nw791 nw787 vdd vdd pch w=2u l=180n
CT2351 t2351 0 0.1f
M6283 nw791 nw788 t2351 0 nch w=1u l=180n
M6284 t2351 nw787 0 0 nch w=1u l=180n
Cnw791 nw791 0 2f
M6285 nw792 nw790 vdd vdd pch w=2u l=180n
M6286 nw792 nw791 vdd vdd pch w=2u l=180n
CT2352 t2352 0 0.1f
M6287 nw792 nw790 t2352 0 nch w=1u l=180n
M6288 t2352 nw791 0 0 nch w=1u l=180n
Cnw792 nw792 0 2f
CT2353 t2353 0 0.1f
CT2354 t2354 0 0.1f
CT2355 t2355 0 0.1f
M6289 t2353 nw129 vdd vdd pch w=2u l=180n
M6290 t2353 nw719 vdd vdd pch w=2u l=180n
CT2356 t2356 0 0.1f
M6291 t2353 nw129 t2356 0 nch w=1u l=180n
M6292 t2356 nw719 0 0 nch w=1u l=180n
M6293 t2354 nw129 vdd vdd pch w=2u l=180n
M6294 t2354 t2353 vdd vdd pch w=2u l=180n
CT2357 t2357 0 0.1f
M6295 t2354 nw129 t2357 0 nch w=1u l=180n
M6296 t2357 t2353 0 0 nch w=1u l=180n
M6297 t2355 nw719 vdd vdd pch w=2u l=180n
M6298 t2355 t2353 vdd vdd pch w=2u l=180n
CT2358 t2358 0 0.1f
M6299 t2355 nw719 t2358 0 nch w=1u l=180n
M6300 t2358 t2353 0 0 nch w=1u l=180n
M6301 nw793 t2354 vdd vdd pch w=2u l=180n
M6302 nw793 t2355 vdd vdd pch w=2u l=180n
CT2359 t2359 0 0.1f
M6303 nw793 t2354 t2359 0 nch w=1u l=180n
M6304 t2359 t2355 0 0 nch w=1u l=180n
Cnw793 nw793 0 2f
CT2360 t2360 0 0.1f
M6305 t2360 nw129 vdd vdd pch w=2u l=180n
M6306 t2360 nw719 vdd vdd pch w=2u l=180n
CT2361 t2361 0 0.1f
M6307 t2360 nw129 t2361 0 nch w=1u l=180n
M6308 t2361 nw719 0 0 nch w=1u l=180n
M6309 nw794 t2360 vdd vdd pch w=2u l=180n
M6310 nw794 t2360 0 0 nch w=1u l=180n
Cnw794 nw794 0 2f
CT2362 t2362 0 0.1f
CT2363 t2363 0 0.1f
CT2364 t2364 0 0.1f
M6311 t2362 nw130 vdd vdd pch w=2u l=180n
M6312 t2362 nw724 vdd vdd pch w=2u l=180n
CT2365 t2365 0 0.1f
M6313 t2362 nw130 t2365 0 nch w=1u l=180n
M6314 t2365 nw724 0 0 nch w=1u l=180n
M6315 t2363 nw130 vdd vdd pch w=2u l=180n
M6316 t2363 t2362 vdd vdd pch w=2u l=180n
CT2366 t2366 0 0.1f
M6317 t2363 nw130 t2366 0 nch w=1u l=180n
M6318 t2366 t2362 0 0 nch w=1u l=180n
M6319 t2364 nw724 vdd vdd pch w=2u l=180n
M6320 t2364 t2362 vdd vdd pch w=2u l=180n
CT2367 t2367 0 0.1f
M6321 t2364 nw724 t2367 0 nch w=1u l=180n
M6322 t2367 t2362 0 0 nch w=1u l=180n
M6323 nw795 t2363 vdd vdd pch w=2u l=180n
M6324 nw795 t2364 vdd vdd pch w=2u l=180n
CT2368 t2368 0 0.1f
M6325 nw795 t2363 t2368 0 nch w=1u l=180n
M6326 t2368 t2364 0 0 nch w=1u l=180n
Cnw795 nw795 0 2f
CT2369 t2369 0 0.1f
CT2370 t2370 0 0.1f
CT2371 t2371 0 0.1f
M6327 t2369 nw795 vdd vdd pch w=2u l=180n
M6328 t2369 nw794 vdd vdd pch w=2u l=180n
CT2372 t2372 0 0.1f
M6329 t2369 nw795 t2372 0 nch w=1u l=180n
M6330 t2372 nw794 0 0 nch w=1u l=180n
M6331 t2370 nw795 vdd vdd pch w=2u l=180n
M6332 t2370 t2369 vdd vdd pch w=2u l=180n
CT2373 t2373 0 0.1f
M6333 t2370 nw795 t2373 0 nch w=1u l=180n
M6334 t2373 t2369 0 0 nch w=1u l=180n
M6335 t2371 nw794 vdd vdd pch w=2u l=180n
M6336 t2371 t2369 vdd vdd pch w=2u l=180n
CT2374 t2374 0 0.1f
M6337 t2371 nw794 t2374 0 nch w=1u l=180n
M6338 t2374 t2369 0 0 nch w=1u l=180n
M6339 nw796 t2370 vdd vdd pch w=2u l=180n
M6340 nw796 t2371 vdd vdd pch w=2u l=180n
CT2375 t2375 0 0.1f
M6341 nw796 t2370 t2375 0 nch w=1u l=180n
M6342 t2375 t2371 0 0 nch w=1u l=180n
Cnw796 nw796 0 2f
M6343 nw797 nw130 vdd vdd pch w=2u l=180n
M6344 nw797 nw724 vdd vdd pch w=2u l=180n
CT2376 t2376 0 0.1f
M6345 nw797 nw130 t2376 0 nch w=1u l=180n
M6346 t2376 nw724 0 0 nch w=1u l=180n
Cnw797 nw797 0 2f
M6347 nw798 nw795 vdd vdd pch w=2u l=180n
M6348 nw798 nw794 vdd vdd pch w=2u l=180n
CT2377 t2377 0 0.1f
M6349 nw798 nw795 t2377 0 nch w=1u l=180n
M6350 t2377 nw794 0 0 nch w=1u l=180n
Cnw798 nw798 0 2f
M6351 nw799 nw797 vdd vdd pch w=2u l=180n
M6352 nw799 nw798 vdd vdd pch w=2u l=180n
CT2378 t2378 0 0.1f
M6353 nw799 nw797 t2378 0 nch w=1u l=180n
M6354 t2378 nw798 0 0 nch w=1u l=180n
Cnw799 nw799 0 2f
CT2379 t2379 0 0.1f
CT2380 t2380 0 0.1f
CT2381 t2381 0 0.1f
M6355 t2379 nw131 vdd vdd pch w=2u l=180n
M6356 t2379 nw729 vdd vdd pch w=2u l=180n
CT2382 t2382 0 0.1f
M6357 t2379 nw131 t2382 0 nch w=1u l=180n
M6358 t2382 nw729 0 0 nch w=1u l=180n
M6359 t2380 nw131 vdd vdd pch w=2u l=180n
M6360 t2380 t2379 vdd vdd pch w=2u l=180n
CT2383 t2383 0 0.1f
M6361 t2380 nw131 t2383 0 nch w=1u l=180n
M6362 t2383 t2379 0 0 nch w=1u l=180n
M6363 t2381 nw729 vdd vdd pch w=2u l=180n
M6364 t2381 t2379 vdd vdd pch w=2u l=180n
CT2384 t2384 0 0.1f
M6365 t2381 nw729 t2384 0 nch w=1u l=180n
M6366 t2384 t2379 0 0 nch w=1u l=180n
M6367 nw800 t2380 vdd vdd pch w=2u l=180n
M6368 nw800 t2381 vdd vdd pch w=2u l=180n
CT2385 t2385 0 0.1f
M6369 nw800 t2380 t2385 0 nch w=1u l=180n
M6370 t2385 t2381 0 0 nch w=1u l=180n
Cnw800 nw800 0 2f
CT2386 t2386 0 0.1f
CT2387 t2387 0 0.1f
CT2388 t2388 0 0.1f
M6371 t2386 nw800 vdd vdd pch w=2u l=180n
M6372 t2386 nw799 vdd vdd pch w=2u l=180n
CT2389 t2389 0 0.1f
M6373 t2386 nw800 t2389 0 nch w=1u l=180n
M6374 t2389 nw799 0 0 nch w=1u l=180n
M6375 t2387 nw800 vdd vdd pch w=2u l=180n
M6376 t2387 t2386 vdd vdd pch w=2u l=180n
CT2390 t2390 0 0.1f
M6377 t2387 nw800 t2390 0 nch w=1u l=180n
M6378 t2390 t2386 0 0 nch w=1u l=180n
M6379 t2388 nw799 vdd vdd pch w=2u l=180n
M6380 t2388 t2386 vdd vdd pch w=2u l=180n
CT2391 t2391 0 0.1f
M6381 t2388 nw799 t2391 0 nch w=1u l=180n
M6382 t2391 t2386 0 0 nch w=1u l=180n
M6383 nw801 t2387 vdd vdd pch w=2u l=180n
M6384 nw801 t2388 vdd vdd pch w=2u l=180n
CT2392 t2392 0 0.1f
M6385 nw801 t2387 t2392 0 nch w=1u l=180n
M6386 t2392 t2388 0 0 nch w=1u l=180n
Cnw801 nw801 0 2f
M6387 nw802 nw131 vdd vdd pch w=2u l=180n
M6388 nw802 nw729 vdd vdd pch w=2u l=180n
CT2393 t2393 0 0.1f
M6389 nw802 nw131 t2393 0 nch w=1u l=180n
M6390 t2393 nw729 0 0 nch w=1u l=180n
Cnw802 nw802 0 2f
M6391 nw803 nw800 vdd vdd pch w=2u l=180n
M6392 nw803 nw799 vdd vdd pch w=2u l=180n
CT2394 t2394 0 0.1f
M6393 nw803 nw800 t2394 0 nch w=1u l=180n
M6394 t2394 nw799 0 0 nch w=1u l=180n
Cnw803 nw803 0 2f
M6395 nw804 nw802 vdd vdd pch w=2u l=180n
M6396 nw804 nw803 vdd vdd pch w=2u l=180n
CT2395 t2395 0 0.1f
M6397 nw804 nw802 t2395 0 nch w=1u l=180n
M6398 t2395 nw803 0 0 nch w=1u l=180n
Cnw804 nw804 0 2f
CT2396 t2396 0 0.1f
CT2397 t2397 0 0.1f
CT2398 t2398 0 0.1f
M6399 t2396 nw132 vdd vdd pch w=2u l=180n
M6400 t2396 nw734 vdd vdd pch w=2u l=180n
CT2399 t2399 0 0.1f
M6401 t2396 nw132 t2399 0 nch w=1u l=180n
M6402 t2399 nw734 0 0 nch w=1u l=180n
M6403 t2397 nw132 vdd vdd pch w=2u l=180n
M6404 t2397 t2396 vdd vdd pch w=2u l=180n
CT2400 t2400 0 0.1f
M6405 t2397 nw132 t2400 0 nch w=1u l=180n
M6406 t2400 t2396 0 0 nch w=1u l=180n
M6407 t2398 nw734 vdd vdd pch w=2u l=180n
M6408 t2398 t2396 vdd vdd pch w=2u l=180n
CT2401 t2401 0 0.1f
M6409 t2398 nw734 t2401 0 nch w=1u l=180n
M6410 t2401 t2396 0 0 nch w=1u l=180n
M6411 nw805 t2397 vdd vdd pch w=2u l=180n
M6412 nw805 t2398 vdd vdd pch w=2u l=180n
CT2402 t2402 0 0.1f
M6413 nw805 t2397 t2402 0 nch w=1u l=180n
M6414 t2402 t2398 0 0 nch w=1u l=180n
Cnw805 nw805 0 2f
CT2403 t2403 0 0.1f
CT2404 t2404 0 0.1f
CT2405 t2405 0 0.1f
M6415 t2403 nw805 vdd vdd pch w=2u l=180n
M6416 t2403 nw804 vdd vdd pch w=2u l=180n
CT2406 t2406 0 0.1f
M6417 t2403 nw805 t2406 0 nch w=1u l=180n
M6418 t2406 nw804 0 0 nch w=1u l=180n
M6419 t2404 nw805 vdd vdd pch w=2u l=180n
M6420 t2404 t2403 vdd vdd pch w=2u l=180n
CT2407 t2407 0 0.1f
M6421 t2404 nw805 t2407 0 nch w=1u l=180n
M6422 t2407 t2403 0 0 nch w=1u l=180n
M6423 t2405 nw804 vdd vdd pch w=2u l=180n
M6424 t2405 t2403 vdd vdd pch w=2u l=180n
CT2408 t2408 0 0.1f
M6425 t2405 nw804 t2408 0 nch w=1u l=180n
M6426 t2408 t2403 0 0 nch w=1u l=180n
M6427 nw806 t2404 vdd vdd pch w=2u l=180n
M6428 nw806 t2405 vdd vdd pch w=2u l=180n
CT2409 t2409 0 0.1f
M6429 nw806 t2404 t2409 0 nch w=1u l=180n
M6430 t2409 t2405 0 0 nch w=1u l=180n
Cnw806 nw806 0 2f
M6431 nw807 nw132 vdd vdd pch w=2u l=180n
M6432 nw807 nw734 vdd vdd pch w=2u l=180n
CT2410 t2410 0 0.1f
M6433 nw807 nw132 t2410 0 nch w=1u l=180n
M6434 t2410 nw734 0 0 nch w=1u l=180n
Cnw807 nw807 0 2f
M6435 nw808 nw805 vdd vdd pch w=2u l=180n
M6436 nw808 nw804 vdd vdd pch w=2u l=180n
CT2411 t2411 0 0.1f
M6437 nw808 nw805 t2411 0 nch w=1u l=180n
M6438 t2411 nw804 0 0 nch w=1u l=180n
Cnw808 nw808 0 2f
M6439 nw809 nw807 vdd vdd pch w=2u l=180n
M6440 nw809 nw808 vdd vdd pch w=2u l=180n
CT2412 t2412 0 0.1f
M6441 nw809 nw807 t2412 0 nch w=1u l=180n
M6442 t2412 nw808 0 0 nch w=1u l=180n
Cnw809 nw809 0 2f
CT2413 t2413 0 0.1f
CT2414 t2414 0 0.1f
CT2415 t2415 0 0.1f
M6443 t2413 nw133 vdd vdd pch w=2u l=180n
M6444 t2413 nw739 vdd vdd pch w=2u l=180n
CT2416 t2416 0 0.1f
M6445 t2413 nw133 t2416 0 nch w=1u l=180n
M6446 t2416 nw739 0 0 nch w=1u l=180n
M6447 t2414 nw133 vdd vdd pch w=2u l=180n
M6448 t2414 t2413 vdd vdd pch w=2u l=180n
CT2417 t2417 0 0.1f
M6449 t2414 nw133 t2417 0 nch w=1u l=180n
M6450 t2417 t2413 0 0 nch w=1u l=180n
M6451 t2415 nw739 vdd vdd pch w=2u l=180n
M6452 t2415 t2413 vdd vdd pch w=2u l=180n
CT2418 t2418 0 0.1f
M6453 t2415 nw739 t2418 0 nch w=1u l=180n
M6454 t2418 t2413 0 0 nch w=1u l=180n
M6455 nw810 t2414 vdd vdd pch w=2u l=180n
M6456 nw810 t2415 vdd vdd pch w=2u l=180n
CT2419 t2419 0 0.1f
M6457 nw810 t2414 t2419 0 nch w=1u l=180n
M6458 t2419 t2415 0 0 nch w=1u l=180n
Cnw810 nw810 0 2f
CT2420 t2420 0 0.1f
CT2421 t2421 0 0.1f
CT2422 t2422 0 0.1f
M6459 t2420 nw810 vdd vdd pch w=2u l=180n
M6460 t2420 nw809 vdd vdd pch w=2u l=180n
CT2423 t2423 0 0.1f
M6461 t2420 nw810 t2423 0 nch w=1u l=180n
M6462 t2423 nw809 0 0 nch w=1u l=180n
M6463 t2421 nw810 vdd vdd pch w=2u l=180n
M6464 t2421 t2420 vdd vdd pch w=2u l=180n
CT2424 t2424 0 0.1f
M6465 t2421 nw810 t2424 0 nch w=1u l=180n
M6466 t2424 t2420 0 0 nch w=1u l=180n
M6467 t2422 nw809 vdd vdd pch w=2u l=180n
M6468 t2422 t2420 vdd vdd pch w=2u l=180n
CT2425 t2425 0 0.1f
M6469 t2422 nw809 t2425 0 nch w=1u l=180n
M6470 t2425 t2420 0 0 nch w=1u l=180n
M6471 nw811 t2421 vdd vdd pch w=2u l=180n
M6472 nw811 t2422 vdd vdd pch w=2u l=180n
CT2426 t2426 0 0.1f
M6473 nw811 t2421 t2426 0 nch w=1u l=180n
M6474 t2426 t2422 0 0 nch w=1u l=180n
Cnw811 nw811 0 2f
M6475 nw812 nw133 vdd vdd pch w=2u l=180n
M6476 nw812 nw739 vdd vdd pch w=2u l=180n
CT2427 t2427 0 0.1f
M6477 nw812 nw133 t2427 0 nch w=1u l=180n
M6478 t2427 nw739 0 0 nch w=1u l=180n
Cnw812 nw812 0 2f
M6479 nw813 nw810 vdd vdd pch w=2u l=180n
M6480 nw813 nw809 vdd vdd pch w=2u l=180n
CT2428 t2428 0 0.1f
M6481 nw813 nw810 t2428 0 nch w=1u l=180n
M6482 t2428 nw809 0 0 nch w=1u l=180n
Cnw813 nw813 0 2f
M6483 nw814 nw812 vdd vdd pch w=2u l=180n
M6484 nw814 nw813 vdd vdd pch w=2u l=180n
CT2429 t2429 0 0.1f
M6485 nw814 nw812 t2429 0 nch w=1u l=180n
M6486 t2429 nw813 0 0 nch w=1u l=180n
Cnw814 nw814 0 2f
CT2430 t2430 0 0.1f
CT2431 t2431 0 0.1f
CT2432 t2432 0 0.1f
M6487 t2430 nw134 vdd vdd pch w=2u l=180n
M6488 t2430 nw744 vdd vdd pch w=2u l=180n
CT2433 t2433 0 0.1f
M6489 t2430 nw134 t2433 0 nch w=1u l=180n
M6490 t2433 nw744 0 0 nch w=1u l=180n
M6491 t2431 nw134 vdd vdd pch w=2u l=180n
M6492 t2431 t2430 vdd vdd pch w=2u l=180n
CT2434 t2434 0 0.1f
M6493 t2431 nw134 t2434 0 nch w=1u l=180n
M6494 t2434 t2430 0 0 nch w=1u l=180n
M6495 t2432 nw744 vdd vdd pch w=2u l=180n
M6496 t2432 t2430 vdd vdd pch w=2u l=180n
CT2435 t2435 0 0.1f
M6497 t2432 nw744 t2435 0 nch w=1u l=180n
M6498 t2435 t2430 0 0 nch w=1u l=180n
M6499 nw815 t2431 vdd vdd pch w=2u l=180n
M6500 nw815 t2432 vdd vdd pch w=2u l=180n
CT2436 t2436 0 0.1f
M6501 nw815 t2431 t2436 0 nch w=1u l=180n
M6502 t2436 t2432 0 0 nch w=1u l=180n
Cnw815 nw815 0 2f
CT2437 t2437 0 0.1f
CT2438 t2438 0 0.1f
CT2439 t2439 0 0.1f
M6503 t2437 nw815 vdd vdd pch w=2u l=180n
M6504 t2437 nw814 vdd vdd pch w=2u l=180n
CT2440 t2440 0 0.1f
M6505 t2437 nw815 t2440 0 nch w=1u l=180n
M6506 t2440 nw814 0 0 nch w=1u l=180n
M6507 t2438 nw815 vdd vdd pch w=2u l=180n
M6508 t2438 t2437 vdd vdd pch w=2u l=180n
CT2441 t2441 0 0.1f
M6509 t2438 nw815 t2441 0 nch w=1u l=180n
M6510 t2441 t2437 0 0 nch w=1u l=180n
M6511 t2439 nw814 vdd vdd pch w=2u l=180n
M6512 t2439 t2437 vdd vdd pch w=2u l=180n
CT2442 t2442 0 0.1f
M6513 t2439 nw814 t2442 0 nch w=1u l=180n
M6514 t2442 t2437 0 0 nch w=1u l=180n
M6515 nw816 t2438 vdd vdd pch w=2u l=180n
M6516 nw816 t2439 vdd vdd pch w=2u l=180n
CT2443 t2443 0 0.1f
M6517 nw816 t2438 t2443 0 nch w=1u l=180n
M6518 t2443 t2439 0 0 nch w=1u l=180n
Cnw816 nw816 0 2f
M6519 nw817 nw134 vdd vdd pch w=2u l=180n
M6520 nw817 nw744 vdd vdd pch w=2u l=180n
CT2444 t2444 0 0.1f
M6521 nw817 nw134 t2444 0 nch w=1u l=180n
M6522 t2444 nw744 0 0 nch w=1u l=180n
Cnw817 nw817 0 2f
M6523 nw818 nw815 vdd vdd pch w=2u l=180n
M6524 nw818 nw814 vdd vdd pch w=2u l=180n
CT2445 t2445 0 0.1f
M6525 nw818 nw815 t2445 0 nch w=1u l=180n
M6526 t2445 nw814 0 0 nch w=1u l=180n
Cnw818 nw818 0 2f
M6527 nw819 nw817 vdd vdd pch w=2u l=180n
M6528 nw819 nw818 vdd vdd pch w=2u l=180n
CT2446 t2446 0 0.1f
M6529 nw819 nw817 t2446 0 nch w=1u l=180n
M6530 t2446 nw818 0 0 nch w=1u l=180n
Cnw819 nw819 0 2f
CT2447 t2447 0 0.1f
CT2448 t2448 0 0.1f
CT2449 t2449 0 0.1f
M6531 t2447 nw135 vdd vdd pch w=2u l=180n
M6532 t2447 nw749 vdd vdd pch w=2u l=180n
CT2450 t2450 0 0.1f
M6533 t2447 nw135 t2450 0 nch w=1u l=180n
M6534 t2450 nw749 0 0 nch w=1u l=180n
M6535 t2448 nw135 vdd vdd pch w=2u l=180n
M6536 t2448 t2447 vdd vdd pch w=2u l=180n
CT2451 t2451 0 0.1f
M6537 t2448 nw135 t2451 0 nch w=1u l=180n
M6538 t2451 t2447 0 0 nch w=1u l=180n
M6539 t2449 nw749 vdd vdd pch w=2u l=180n
M6540 t2449 t2447 vdd vdd pch w=2u l=180n
CT2452 t2452 0 0.1f
M6541 t2449 nw749 t2452 0 nch w=1u l=180n
M6542 t2452 t2447 0 0 nch w=1u l=180n
M6543 nw820 t2448 vdd vdd pch w=2u l=180n
M6544 nw820 t2449 vdd vdd pch w=2u l=180n
CT2453 t2453 0 0.1f
M6545 nw820 t2448 t2453 0 nch w=1u l=180n
M6546 t2453 t2449 0 0 nch w=1u l=180n
Cnw820 nw820 0 2f
CT2454 t2454 0 0.1f
CT2455 t2455 0 0.1f
CT2456 t2456 0 0.1f
M6547 t2454 nw820 vdd vdd pch w=2u l=180n
M6548 t2454 nw819 vdd vdd pch w=2u l=180n
CT2457 t2457 0 0.1f
M6549 t2454 nw820 t2457 0 nch w=1u l=180n
M6550 t2457 nw819 0 0 nch w=1u l=180n
M6551 t2455 nw820 vdd vdd pch w=2u l=180n
M6552 t2455 t2454 vdd vdd pch w=2u l=180n
CT2458 t2458 0 0.1f
M6553 t2455 nw820 t2458 0 nch w=1u l=180n
M6554 t2458 t2454 0 0 nch w=1u l=180n
M6555 t2456 nw819 vdd vdd pch w=2u l=180n
M6556 t2456 t2454 vdd vdd pch w=2u l=180n
CT2459 t2459 0 0.1f
M6557 t2456 nw819 t2459 0 nch w=1u l=180n
M6558 t2459 t2454 0 0 nch w=1u l=180n
M6559 nw821 t2455 vdd vdd pch w=2u l=180n
M6560 nw821 t2456 vdd vdd pch w=2u l=180n
CT2460 t2460 0 0.1f
M6561 nw821 t2455 t2460 0 nch w=1u l=180n
M6562 t2460 t2456 0 0 nch w=1u l=180n
Cnw821 nw821 0 2f
M6563 nw822 nw135 vdd vdd pch w=2u l=180n
M6564 nw822 nw749 vdd vdd pch w=2u l=180n
CT2461 t2461 0 0.1f
M6565 nw822 nw135 t2461 0 nch w=1u l=180n
M6566 t2461 nw749 0 0 nch w=1u l=180n
Cnw822 nw822 0 2f
M6567 nw823 nw820 vdd vdd pch w=2u l=180n
M6568 nw823 nw819 vdd vdd pch w=2u l=180n
CT2462 t2462 0 0.1f
M6569 nw823 nw820 t2462 0 nch w=1u l=180n
M6570 t2462 nw819 0 0 nch w=1u l=180n
Cnw823 nw823 0 2f
M6571 nw824 nw822 vdd vdd pch w=2u l=180n
M6572 nw824 nw823 vdd vdd pch w=2u l=180n
CT2463 t2463 0 0.1f
M6573 nw824 nw822 t2463 0 nch w=1u l=180n
M6574 t2463 nw823 0 0 nch w=1u l=180n
Cnw824 nw824 0 2f
CT2464 t2464 0 0.1f
CT2465 t2465 0 0.1f
CT2466 t2466 0 0.1f
M6575 t2464 nw136 vdd vdd pch w=2u l=180n
M6576 t2464 nw754 vdd vdd pch w=2u l=180n
CT2467 t2467 0 0.1f
M6577 t2464 nw136 t2467 0 nch w=1u l=180n
M6578 t2467 nw754 0 0 nch w=1u l=180n
M6579 t2465 nw136 vdd vdd pch w=2u l=180n
M6580 t2465 t2464 vdd vdd pch w=2u l=180n
CT2468 t2468 0 0.1f
M6581 t2465 nw136 t2468 0 nch w=1u l=180n
M6582 t2468 t2464 0 0 nch w=1u l=180n
M6583 t2466 nw754 vdd vdd pch w=2u l=180n
M6584 t2466 t2464 vdd vdd pch w=2u l=180n
CT2469 t2469 0 0.1f
M6585 t2466 nw754 t2469 0 nch w=1u l=180n
M6586 t2469 t2464 0 0 nch w=1u l=180n
M6587 nw825 t2465 vdd vdd pch w=2u l=180n
M6588 nw825 t2466 vdd vdd pch w=2u l=180n
CT2470 t2470 0 0.1f
M6589 nw825 t2465 t2470 0 nch w=1u l=180n
M6590 t2470 t2466 0 0 nch w=1u l=180n
Cnw825 nw825 0 2f
CT2471 t2471 0 0.1f
CT2472 t2472 0 0.1f
CT2473 t2473 0 0.1f
M6591 t2471 nw825 vdd vdd pch w=2u l=180n
M6592 t2471 nw824 vdd vdd pch w=2u l=180n
CT2474 t2474 0 0.1f
M6593 t2471 nw825 t2474 0 nch w=1u l=180n
M6594 t2474 nw824 0 0 nch w=1u l=180n
M6595 t2472 nw825 vdd vdd pch w=2u l=180n
M6596 t2472 t2471 vdd vdd pch w=2u l=180n
CT2475 t2475 0 0.1f
M6597 t2472 nw825 t2475 0 nch w=1u l=180n
M6598 t2475 t2471 0 0 nch w=1u l=180n
M6599 t2473 nw824 vdd vdd pch w=2u l=180n
M6600 t2473 t2471 vdd vdd pch w=2u l=180n
CT2476 t2476 0 0.1f
M6601 t2473 nw824 t2476 0 nch w=1u l=180n
M6602 t2476 t2471 0 0 nch w=1u l=180n
M6603 nw826 t2472 vdd vdd pch w=2u l=180n
M6604 nw826 t2473 vdd vdd pch w=2u l=180n
CT2477 t2477 0 0.1f
M6605 nw826 t2472 t2477 0 nch w=1u l=180n
M6606 t2477 t2473 0 0 nch w=1u l=180n
Cnw826 nw826 0 2f
M6607 nw827 nw136 vdd vdd pch w=2u l=180n
M6608 nw827 nw754 vdd vdd pch w=2u l=180n
CT2478 t2478 0 0.1f
M6609 nw827 nw136 t2478 0 nch w=1u l=180n
M6610 t2478 nw754 0 0 nch w=1u l=180n
Cnw827 nw827 0 2f
M6611 nw828 nw825 vdd vdd pch w=2u l=180n
M6612 nw828 nw824 vdd vdd pch w=2u l=180n
CT2479 t2479 0 0.1f
M6613 nw828 nw825 t2479 0 nch w=1u l=180n
M6614 t2479 nw824 0 0 nch w=1u l=180n
Cnw828 nw828 0 2f
M6615 nw829 nw827 vdd vdd pch w=2u l=180n
M6616 nw829 nw828 vdd vdd pch w=2u l=180n
CT2480 t2480 0 0.1f
M6617 nw829 nw827 t2480 0 nch w=1u l=180n
M6618 t2480 nw828 0 0 nch w=1u l=180n
Cnw829 nw829 0 2f
CT2481 t2481 0 0.1f
CT2482 t2482 0 0.1f
CT2483 t2483 0 0.1f
M6619 t2481 nw137 vdd vdd pch w=2u l=180n
M6620 t2481 nw759 vdd vdd pch w=2u l=180n
CT2484 t2484 0 0.1f
M6621 t2481 nw137 t2484 0 nch w=1u l=180n
M6622 t2484 nw759 0 0 nch w=1u l=180n
M6623 t2482 nw137 vdd vdd pch w=2u l=180n
M6624 t2482 t2481 vdd vdd pch w=2u l=180n
CT2485 t2485 0 0.1f
M6625 t2482 nw137 t2485 0 nch w=1u l=180n
M6626 t2485 t2481 0 0 nch w=1u l=180n
M6627 t2483 nw759 vdd vdd pch w=2u l=180n
M6628 t2483 t2481 vdd vdd pch w=2u l=180n
CT2486 t2486 0 0.1f
M6629 t2483 nw759 t2486 0 nch w=1u l=180n
M6630 t2486 t2481 0 0 nch w=1u l=180n
M6631 nw830 t2482 vdd vdd pch w=2u l=180n
M6632 nw830 t2483 vdd vdd pch w=2u l=180n
CT2487 t2487 0 0.1f
M6633 nw830 t2482 t2487 0 nch w=1u l=180n
M6634 t2487 t2483 0 0 nch w=1u l=180n
Cnw830 nw830 0 2f
CT2488 t2488 0 0.1f
CT2489 t2489 0 0.1f
CT2490 t2490 0 0.1f
M6635 t2488 nw830 vdd vdd pch w=2u l=180n
M6636 t2488 nw829 vdd vdd pch w=2u l=180n
CT2491 t2491 0 0.1f
M6637 t2488 nw830 t2491 0 nch w=1u l=180n
M6638 t2491 nw829 0 0 nch w=1u l=180n
M6639 t2489 nw830 vdd vdd pch w=2u l=180n
M6640 t2489 t2488 vdd vdd pch w=2u l=180n
CT2492 t2492 0 0.1f
M6641 t2489 nw830 t2492 0 nch w=1u l=180n
M6642 t2492 t2488 0 0 nch w=1u l=180n
M6643 t2490 nw829 vdd vdd pch w=2u l=180n
M6644 t2490 t2488 vdd vdd pch w=2u l=180n
CT2493 t2493 0 0.1f
M6645 t2490 nw829 t2493 0 nch w=1u l=180n
M6646 t2493 t2488 0 0 nch w=1u l=180n
M6647 nw831 t2489 vdd vdd pch w=2u l=180n
M6648 nw831 t2490 vdd vdd pch w=2u l=180n
CT2494 t2494 0 0.1f
M6649 nw831 t2489 t2494 0 nch w=1u l=180n
M6650 t2494 t2490 0 0 nch w=1u l=180n
Cnw831 nw831 0 2f
M6651 nw832 nw137 vdd vdd pch w=2u l=180n
M6652 nw832 nw759 vdd vdd pch w=2u l=180n
CT2495 t2495 0 0.1f
M6653 nw832 nw137 t2495 0 nch w=1u l=180n
M6654 t2495 nw759 0 0 nch w=1u l=180n
Cnw832 nw832 0 2f
M6655 nw833 nw830 vdd vdd pch w=2u l=180n
M6656 nw833 nw829 vdd vdd pch w=2u l=180n
CT2496 t2496 0 0.1f
M6657 nw833 nw830 t2496 0 nch w=1u l=180n
M6658 t2496 nw829 0 0 nch w=1u l=180n
Cnw833 nw833 0 2f
M6659 nw834 nw832 vdd vdd pch w=2u l=180n
M6660 nw834 nw833 vdd vdd pch w=2u l=180n
CT2497 t2497 0 0.1f
M6661 nw834 nw832 t2497 0 nch w=1u l=180n
M6662 t2497 nw833 0 0 nch w=1u l=180n
Cnw834 nw834 0 2f
CT2498 t2498 0 0.1f
CT2499 t2499 0 0.1f
CT2500 t2500 0 0.1f
M6663 t2498 nw138 vdd vdd pch w=2u l=180n
M6664 t2498 nw764 vdd vdd pch w=2u l=180n
CT2501 t2501 0 0.1f
M6665 t2498 nw138 t2501 0 nch w=1u l=180n
M6666 t2501 nw764 0 0 nch w=1u l=180n
M6667 t2499 nw138 vdd vdd pch w=2u l=180n
M6668 t2499 t2498 vdd vdd pch w=2u l=180n
CT2502 t2502 0 0.1f
M6669 t2499 nw138 t2502 0 nch w=1u l=180n
M6670 t2502 t2498 0 0 nch w=1u l=180n
M6671 t2500 nw764 vdd vdd pch w=2u l=180n
M6672 t2500 t2498 vdd vdd pch w=2u l=180n
CT2503 t2503 0 0.1f
M6673 t2500 nw764 t2503 0 nch w=1u l=180n
M6674 t2503 t2498 0 0 nch w=1u l=180n
M6675 nw835 t2499 vdd vdd pch w=2u l=180n
M6676 nw835 t2500 vdd vdd pch w=2u l=180n
CT2504 t2504 0 0.1f
M6677 nw835 t2499 t2504 0 nch w=1u l=180n
M6678 t2504 t2500 0 0 nch w=1u l=180n
Cnw835 nw835 0 2f
CT2505 t2505 0 0.1f
CT2506 t2506 0 0.1f
CT2507 t2507 0 0.1f
M6679 t2505 nw835 vdd vdd pch w=2u l=180n
M6680 t2505 nw834 vdd vdd pch w=2u l=180n
CT2508 t2508 0 0.1f
M6681 t2505 nw835 t2508 0 nch w=1u l=180n
M6682 t2508 nw834 0 0 nch w=1u l=180n
M6683 t2506 nw835 vdd vdd pch w=2u l=180n
M6684 t2506 t2505 vdd vdd pch w=2u l=180n
CT2509 t2509 0 0.1f
M6685 t2506 nw835 t2509 0 nch w=1u l=180n
M6686 t2509 t2505 0 0 nch w=1u l=180n
M6687 t2507 nw834 vdd vdd pch w=2u l=180n
M6688 t2507 t2505 vdd vdd pch w=2u l=180n
CT2510 t2510 0 0.1f
M6689 t2507 nw834 t2510 0 nch w=1u l=180n
M6690 t2510 t2505 0 0 nch w=1u l=180n
M6691 nw836 t2506 vdd vdd pch w=2u l=180n
M6692 nw836 t2507 vdd vdd pch w=2u l=180n
CT2511 t2511 0 0.1f
M6693 nw836 t2506 t2511 0 nch w=1u l=180n
M6694 t2511 t2507 0 0 nch w=1u l=180n
Cnw836 nw836 0 2f
M6695 nw837 nw138 vdd vdd pch w=2u l=180n
M6696 nw837 nw764 vdd vdd pch w=2u l=180n
CT2512 t2512 0 0.1f
M6697 nw837 nw138 t2512 0 nch w=1u l=180n
M6698 t2512 nw764 0 0 nch w=1u l=180n
Cnw837 nw837 0 2f
M6699 nw838 nw835 vdd vdd pch w=2u l=180n
M6700 nw838 nw834 vdd vdd pch w=2u l=180n
CT2513 t2513 0 0.1f
M6701 nw838 nw835 t2513 0 nch w=1u l=180n
M6702 t2513 nw834 0 0 nch w=1u l=180n
Cnw838 nw838 0 2f
M6703 nw839 nw837 vdd vdd pch w=2u l=180n
M6704 nw839 nw838 vdd vdd pch w=2u l=180n
CT2514 t2514 0 0.1f
M6705 nw839 nw837 t2514 0 nch w=1u l=180n
M6706 t2514 nw838 0 0 nch w=1u l=180n
Cnw839 nw839 0 2f
CT2515 t2515 0 0.1f
CT2516 t2516 0 0.1f
CT2517 t2517 0 0.1f
M6707 t2515 nw139 vdd vdd pch w=2u l=180n
M6708 t2515 nw769 vdd vdd pch w=2u l=180n
CT2518 t2518 0 0.1f
M6709 t2515 nw139 t2518 0 nch w=1u l=180n
M6710 t2518 nw769 0 0 nch w=1u l=180n
M6711 t2516 nw139 vdd vdd pch w=2u l=180n
M6712 t2516 t2515 vdd vdd pch w=2u l=180n
CT2519 t2519 0 0.1f
M6713 t2516 nw139 t2519 0 nch w=1u l=180n
M6714 t2519 t2515 0 0 nch w=1u l=180n
M6715 t2517 nw769 vdd vdd pch w=2u l=180n
M6716 t2517 t2515 vdd vdd pch w=2u l=180n
CT2520 t2520 0 0.1f
M6717 t2517 nw769 t2520 0 nch w=1u l=180n
M6718 t2520 t2515 0 0 nch w=1u l=180n
M6719 nw840 t2516 vdd vdd pch w=2u l=180n
M6720 nw840 t2517 vdd vdd pch w=2u l=180n
CT2521 t2521 0 0.1f
M6721 nw840 t2516 t2521 0 nch w=1u l=180n
M6722 t2521 t2517 0 0 nch w=1u l=180n
Cnw840 nw840 0 2f
CT2522 t2522 0 0.1f
CT2523 t2523 0 0.1f
CT2524 t2524 0 0.1f
M6723 t2522 nw840 vdd vdd pch w=2u l=180n
M6724 t2522 nw839 vdd vdd pch w=2u l=180n
CT2525 t2525 0 0.1f
M6725 t2522 nw840 t2525 0 nch w=1u l=180n
M6726 t2525 nw839 0 0 nch w=1u l=180n
M6727 t2523 nw840 vdd vdd pch w=2u l=180n
M6728 t2523 t2522 vdd vdd pch w=2u l=180n
CT2526 t2526 0 0.1f
M6729 t2523 nw840 t2526 0 nch w=1u l=180n
M6730 t2526 t2522 0 0 nch w=1u l=180n
M6731 t2524 nw839 vdd vdd pch w=2u l=180n
M6732 t2524 t2522 vdd vdd pch w=2u l=180n
CT2527 t2527 0 0.1f
M6733 t2524 nw839 t2527 0 nch w=1u l=180n
M6734 t2527 t2522 0 0 nch w=1u l=180n
M6735 nw841 t2523 vdd vdd pch w=2u l=180n
M6736 nw841 t2524 vdd vdd pch w=2u l=180n
CT2528 t2528 0 0.1f
M6737 nw841 t2523 t2528 0 nch w=1u l=180n
M6738 t2528 t2524 0 0 nch w=1u l=180n
Cnw841 nw841 0 2f
M6739 nw842 nw139 vdd vdd pch w=2u l=180n
M6740 nw842 nw769 vdd vdd pch w=2u l=180n
CT2529 t2529 0 0.1f
M6741 nw842 nw139 t2529 0 nch w=1u l=180n
M6742 t2529 nw769 0 0 nch w=1u l=180n
Cnw842 nw842 0 2f
M6743 nw843 nw840 vdd vdd pch w=2u l=180n
M6744 nw843 nw839 vdd vdd pch w=2u l=180n
CT2530 t2530 0 0.1f
M6745 nw843 nw840 t2530 0 nch w=1u l=180n
M6746 t2530 nw839 0 0 nch w=1u l=180n
Cnw843 nw843 0 2f
M6747 nw844 nw842 vdd vdd pch w=2u l=180n
M6748 nw844 nw843 vdd vdd pch w=2u l=180n
CT2531 t2531 0 0.1f
M6749 nw844 nw842 t2531 0 nch w=1u l=180n
M6750 t2531 nw843 0 0 nch w=1u l=180n
Cnw844 nw844 0 2f
CT2532 t2532 0 0.1f
CT2533 t2533 0 0.1f
CT2534 t2534 0 0.1f
M6751 t2532 nw140 vdd vdd pch w=2u l=180n
M6752 t2532 nw774 vdd vdd pch w=2u l=180n
CT2535 t2535 0 0.1f
M6753 t2532 nw140 t2535 0 nch w=1u l=180n
M6754 t2535 nw774 0 0 nch w=1u l=180n
M6755 t2533 nw140 vdd vdd pch w=2u l=180n
M6756 t2533 t2532 vdd vdd pch w=2u l=180n
CT2536 t2536 0 0.1f
M6757 t2533 nw140 t2536 0 nch w=1u l=180n
M6758 t2536 t2532 0 0 nch w=1u l=180n
M6759 t2534 nw774 vdd vdd pch w=2u l=180n
M6760 t2534 t2532 vdd vdd pch w=2u l=180n
CT2537 t2537 0 0.1f
M6761 t2534 nw774 t2537 0 nch w=1u l=180n
M6762 t2537 t2532 0 0 nch w=1u l=180n
M6763 nw845 t2533 vdd vdd pch w=2u l=180n
M6764 nw845 t2534 vdd vdd pch w=2u l=180n
CT2538 t2538 0 0.1f
M6765 nw845 t2533 t2538 0 nch w=1u l=180n
M6766 t2538 t2534 0 0 nch w=1u l=180n
Cnw845 nw845 0 2f
CT2539 t2539 0 0.1f
CT2540 t2540 0 0.1f
CT2541 t2541 0 0.1f
M6767 t2539 nw845 vdd vdd pch w=2u l=180n
M6768 t2539 nw844 vdd vdd pch w=2u l=180n
CT2542 t2542 0 0.1f
M6769 t2539 nw845 t2542 0 nch w=1u l=180n
M6770 t2542 nw844 0 0 nch w=1u l=180n
M6771 t2540 nw845 vdd vdd pch w=2u l=180n
M6772 t2540 t2539 vdd vdd pch w=2u l=180n
CT2543 t2543 0 0.1f
M6773 t2540 nw845 t2543 0 nch w=1u l=180n
M6774 t2543 t2539 0 0 nch w=1u l=180n
M6775 t2541 nw844 vdd vdd pch w=2u l=180n
M6776 t2541 t2539 vdd vdd pch w=2u l=180n
CT2544 t2544 0 0.1f
M6777 t2541 nw844 t2544 0 nch w=1u l=180n
M6778 t2544 t2539 0 0 nch w=1u l=180n
M6779 nw846 t2540 vdd vdd pch w=2u l=180n
M6780 nw846 t2541 vdd vdd pch w=2u l=180n
CT2545 t2545 0 0.1f
M6781 nw846 t2540 t2545 0 nch w=1u l=180n
M6782 t2545 t2541 0 0 nch w=1u l=180n
Cnw846 nw846 0 2f
M6783 nw847 nw140 vdd vdd pch w=2u l=180n
M6784 nw847 nw774 vdd vdd pch w=2u l=180n
CT2546 t2546 0 0.1f
M6785 nw847 nw140 t2546 0 nch w=1u l=180n
M6786 t2546 nw774 0 0 nch w=1u l=180n
Cnw847 nw847 0 2f
M6787 nw848 nw845 vdd vdd pch w=2u l=180n
M6788 nw848 nw844 vdd vdd pch w=2u l=180n
CT2547 t2547 0 0.1f
M6789 nw848 nw845 t2547 0 nch w=1u l=180n
M6790 t2547 nw844 0 0 nch w=1u l=180n
Cnw848 nw848 0 2f
M6791 nw849 nw847 vdd vdd pch w=2u l=180n
M6792 nw849 nw848 vdd vdd pch w=2u l=180n
CT2548 t2548 0 0.1f
M6793 nw849 nw847 t2548 0 nch w=1u l=180n
M6794 t2548 nw848 0 0 nch w=1u l=180n
Cnw849 nw849 0 2f
CT2549 t2549 0 0.1f
CT2550 t2550 0 0.1f
CT2551 t2551 0 0.1f
M6795 t2549 nw141 vdd vdd pch w=2u l=180n
M6796 t2549 nw779 vdd vdd pch w=2u l=180n
CT2552 t2552 0 0.1f
M6797 t2549 nw141 t2552 0 nch w=1u l=180n
M6798 t2552 nw779 0 0 nch w=1u l=180n
M6799 t2550 nw141 vdd vdd pch w=2u l=180n
M6800 t2550 t2549 vdd vdd pch w=2u l=180n
CT2553 t2553 0 0.1f
M6801 t2550 nw141 t2553 0 nch w=1u l=180n
M6802 t2553 t2549 0 0 nch w=1u l=180n
M6803 t2551 nw779 vdd vdd pch w=2u l=180n
M6804 t2551 t2549 vdd vdd pch w=2u l=180n
CT2554 t2554 0 0.1f
M6805 t2551 nw779 t2554 0 nch w=1u l=180n
M6806 t2554 t2549 0 0 nch w=1u l=180n
M6807 nw850 t2550 vdd vdd pch w=2u l=180n
M6808 nw850 t2551 vdd vdd pch w=2u l=180n
CT2555 t2555 0 0.1f
M6809 nw850 t2550 t2555 0 nch w=1u l=180n
M6810 t2555 t2551 0 0 nch w=1u l=180n
Cnw850 nw850 0 2f
CT2556 t2556 0 0.1f
CT2557 t2557 0 0.1f
CT2558 t2558 0 0.1f
M6811 t2556 nw850 vdd vdd pch w=2u l=180n
M6812 t2556 nw849 vdd vdd pch w=2u l=180n
CT2559 t2559 0 0.1f
M6813 t2556 nw850 t2559 0 nch w=1u l=180n
M6814 t2559 nw849 0 0 nch w=1u l=180n
M6815 t2557 nw850 vdd vdd pch w=2u l=180n
M6816 t2557 t2556 vdd vdd pch w=2u l=180n
CT2560 t2560 0 0.1f
M6817 t2557 nw850 t2560 0 nch w=1u l=180n
M6818 t2560 t2556 0 0 nch w=1u l=180n
M6819 t2558 nw849 vdd vdd pch w=2u l=180n
M6820 t2558 t2556 vdd vdd pch w=2u l=180n
CT2561 t2561 0 0.1f
M6821 t2558 nw849 t2561 0 nch w=1u l=180n
M6822 t2561 t2556 0 0 nch w=1u l=180n
M6823 nw851 t2557 vdd vdd pch w=2u l=180n
M6824 nw851 t2558 vdd vdd pch w=2u l=180n
CT2562 t2562 0 0.1f
M6825 nw851 t2557 t2562 0 nch w=1u l=180n
M6826 t2562 t2558 0 0 nch w=1u l=180n
Cnw851 nw851 0 2f
M6827 nw852 nw141 vdd vdd pch w=2u l=180n
M6828 nw852 nw779 vdd vdd pch w=2u l=180n
CT2563 t2563 0 0.1f
M6829 nw852 nw141 t2563 0 nch w=1u l=180n
M6830 t2563 nw779 0 0 nch w=1u l=180n
Cnw852 nw852 0 2f
M6831 nw853 nw850 vdd vdd pch w=2u l=180n
M6832 nw853 nw849 vdd vdd pch w=2u l=180n
CT2564 t2564 0 0.1f
M6833 nw853 nw850 t2564 0 nch w=1u l=180n
M6834 t2564 nw849 0 0 nch w=1u l=180n
Cnw853 nw853 0 2f
M6835 nw854 nw852 vdd vdd pch w=2u l=180n
M6836 nw854 nw853 vdd vdd pch w=2u l=180n
CT2565 t2565 0 0.1f
M6837 nw854 nw852 t2565 0 nch w=1u l=180n
M6838 t2565 nw853 0 0 nch w=1u l=180n
Cnw854 nw854 0 2f
CT2566 t2566 0 0.1f
CT2567 t2567 0 0.1f
CT2568 t2568 0 0.1f
M6839 t2566 nw142 vdd vdd pch w=2u l=180n
M6840 t2566 nw784 vdd vdd pch w=2u l=180n
CT2569 t2569 0 0.1f
M6841 t2566 nw142 t2569 0 nch w=1u l=180n
M6842 t2569 nw784 0 0 nch w=1u l=180n
M6843 t2567 nw142 vdd vdd pch w=2u l=180n
M6844 t2567 t2566 vdd vdd pch w=2u l=180n
CT2570 t2570 0 0.1f
M6845 t2567 nw142 t2570 0 nch w=1u l=180n
M6846 t2570 t2566 0 0 nch w=1u l=180n
M6847 t2568 nw784 vdd vdd pch w=2u l=180n
M6848 t2568 t2566 vdd vdd pch w=2u l=180n
CT2571 t2571 0 0.1f
M6849 t2568 nw784 t2571 0 nch w=1u l=180n
M6850 t2571 t2566 0 0 nch w=1u l=180n
M6851 nw855 t2567 vdd vdd pch w=2u l=180n
M6852 nw855 t2568 vdd vdd pch w=2u l=180n
CT2572 t2572 0 0.1f
M6853 nw855 t2567 t2572 0 nch w=1u l=180n
M6854 t2572 t2568 0 0 nch w=1u l=180n
Cnw855 nw855 0 2f
CT2573 t2573 0 0.1f
CT2574 t2574 0 0.1f
CT2575 t2575 0 0.1f
M6855 t2573 nw855 vdd vdd pch w=2u l=180n
M6856 t2573 nw854 vdd vdd pch w=2u l=180n
CT2576 t2576 0 0.1f
M6857 t2573 nw855 t2576 0 nch w=1u l=180n
M6858 t2576 nw854 0 0 nch w=1u l=180n
M6859 t2574 nw855 vdd vdd pch w=2u l=180n
M6860 t2574 t2573 vdd vdd pch w=2u l=180n
CT2577 t2577 0 0.1f
M6861 t2574 nw855 t2577 0 nch w=1u l=180n
M6862 t2577 t2573 0 0 nch w=1u l=180n
M6863 t2575 nw854 vdd vdd pch w=2u l=180n
M6864 t2575 t2573 vdd vdd pch w=2u l=180n
CT2578 t2578 0 0.1f
M6865 t2575 nw854 t2578 0 nch w=1u l=180n
M6866 t2578 t2573 0 0 nch w=1u l=180n
M6867 nw856 t2574 vdd vdd pch w=2u l=180n
M6868 nw856 t2575 vdd vdd pch w=2u l=180n
CT2579 t2579 0 0.1f
M6869 nw856 t2574 t2579 0 nch w=1u l=180n
M6870 t2579 t2575 0 0 nch w=1u l=180n
Cnw856 nw856 0 2f
M6871 nw857 nw142 vdd vdd pch w=2u l=180n
M6872 nw857 nw784 vdd vdd pch w=2u l=180n
CT2580 t2580 0 0.1f
M6873 nw857 nw142 t2580 0 nch w=1u l=180n
M6874 t2580 nw784 0 0 nch w=1u l=180n
Cnw857 nw857 0 2f
M6875 nw858 nw855 vdd vdd pch w=2u l=180n
M6876 nw858 nw854 vdd vdd pch w=2u l=180n
CT2581 t2581 0 0.1f
M6877 nw858 nw855 t2581 0 nch w=1u l=180n
M6878 t2581 nw854 0 0 nch w=1u l=180n
Cnw858 nw858 0 2f
M6879 nw859 nw857 vdd vdd pch w=2u l=180n
M6880 nw859 nw858 vdd vdd pch w=2u l=180n
CT2582 t2582 0 0.1f
M6881 nw859 nw857 t2582 0 nch w=1u l=180n
M6882 t2582 nw858 0 0 nch w=1u l=180n
Cnw859 nw859 0 2f
CT2583 t2583 0 0.1f
CT2584 t2584 0 0.1f
CT2585 t2585 0 0.1f
M6883 t2583 nw143 vdd vdd pch w=2u l=180n
M6884 t2583 nw789 vdd vdd pch w=2u l=180n
CT2586 t2586 0 0.1f
M6885 t2583 nw143 t2586 0 nch w=1u l=180n
M6886 t2586 nw789 0 0 nch w=1u l=180n
M6887 t2584 nw143 vdd vdd pch w=2u l=180n
M6888 t2584 t2583 vdd vdd pch w=2u l=180n
CT2587 t2587 0 0.1f
M6889 t2584 nw143 t2587 0 nch w=1u l=180n
M6890 t2587 t2583 0 0 nch w=1u l=180n
M6891 t2585 nw789 vdd vdd pch w=2u l=180n
M6892 t2585 t2583 vdd vdd pch w=2u l=180n
CT2588 t2588 0 0.1f
M6893 t2585 nw789 t2588 0 nch w=1u l=180n
M6894 t2588 t2583 0 0 nch w=1u l=180n
M6895 nw860 t2584 vdd vdd pch w=2u l=180n
M6896 nw860 t2585 vdd vdd pch w=2u l=180n
CT2589 t2589 0 0.1f
M6897 nw860 t2584 t2589 0 nch w=1u l=180n
M6898 t2589 t2585 0 0 nch w=1u l=180n
Cnw860 nw860 0 2f
CT2590 t2590 0 0.1f
CT2591 t2591 0 0.1f
CT2592 t2592 0 0.1f
M6899 t2590 nw860 vdd vdd pch w=2u l=180n
M6900 t2590 nw859 vdd vdd pch w=2u l=180n
CT2593 t2593 0 0.1f
M6901 t2590 nw860 t2593 0 nch w=1u l=180n
M6902 t2593 nw859 0 0 nch w=1u l=180n
M6903 t2591 nw860 vdd vdd pch w=2u l=180n
M6904 t2591 t2590 vdd vdd pch w=2u l=180n
CT2594 t2594 0 0.1f
M6905 t2591 nw860 t2594 0 nch w=1u l=180n
M6906 t2594 t2590 0 0 nch w=1u l=180n
M6907 t2592 nw859 vdd vdd pch w=2u l=180n
M6908 t2592 t2590 vdd vdd pch w=2u l=180n
CT2595 t2595 0 0.1f
M6909 t2592 nw859 t2595 0 nch w=1u l=180n
M6910 t2595 t2590 0 0 nch w=1u l=180n
M6911 nw861 t2591 vdd vdd pch w=2u l=180n
M6912 nw861 t2592 vdd vdd pch w=2u l=180n
CT2596 t2596 0 0.1f
M6913 nw861 t2591 t2596 0 nch w=1u l=180n
M6914 t2596 t2592 0 0 nch w=1u l=180n
Cnw861 nw861 0 2f
M6915 nw862 nw143 vdd vdd pch w=2u l=180n
M6916 nw862 nw789 vdd vdd pch w=2u l=180n
CT2597 t2597 0 0.1f
M6917 nw862 nw143 t2597 0 nch w=1u l=180n
M6918 t2597 nw789 0 0 nch w=1u l=180n
Cnw862 nw862 0 2f
M6919 nw863 nw860 vdd vdd pch w=2u l=180n
M6920 nw863 nw859 vdd vdd pch w=2u l=180n
CT2598 t2598 0 0.1f
M6921 nw863 nw860 t2598 0 nch w=1u l=180n
M6922 t2598 nw859 0 0 nch w=1u l=180n
Cnw863 nw863 0 2f
M6923 nw864 nw862 vdd vdd pch w=2u l=180n
M6924 nw864 nw863 vdd vdd pch w=2u l=180n
CT2599 t2599 0 0.1f
M6925 nw864 nw862 t2599 0 nch w=1u l=180n
M6926 t2599 nw863 0 0 nch w=1u l=180n
Cnw864 nw864 0 2f
CT2600 t2600 0 0.1f
CT2601 t2601 0 0.1f
CT2602 t2602 0 0.1f
M6927 t2600 nw144 vdd vdd pch w=2u l=180n
M6928 t2600 nw792 vdd vdd pch w=2u l=180n
CT2603 t2603 0 0.1f
M6929 t2600 nw144 t2603 0 nch w=1u l=180n
M6930 t2603 nw792 0 0 nch w=1u l=180n
M6931 t2601 nw144 vdd vdd pch w=2u l=180n
M6932 t2601 t2600 vdd vdd pch w=2u l=180n
CT2604 t2604 0 0.1f
M6933 t2601 nw144 t2604 0 nch w=1u l=180n
M6934 t2604 t2600 0 0 nch w=1u l=180n
M6935 t2602 nw792 vdd vdd pch w=2u l=180n
M6936 t2602 t2600 vdd vdd pch w=2u l=180n
CT2605 t2605 0 0.1f
M6937 t2602 nw792 t2605 0 nch w=1u l=180n
M6938 t2605 t2600 0 0 nch w=1u l=180n
M6939 nw865 t2601 vdd vdd pch w=2u l=180n
M6940 nw865 t2602 vdd vdd pch w=2u l=180n
CT2606 t2606 0 0.1f
M6941 nw865 t2601 t2606 0 nch w=1u l=180n
M6942 t2606 t2602 0 0 nch w=1u l=180n
Cnw865 nw865 0 2f
CT2607 t2607 0 0.1f
CT2608 t2608 0 0.1f
CT2609 t2609 0 0.1f
M6943 t2607 nw865 vdd vdd pch w=2u l=180n
M6944 t2607 nw864 vdd vdd pch w=2u l=180n
CT2610 t2610 0 0.1f
M6945 t2607 nw865 t2610 0 nch w=1u l=180n
M6946 t2610 nw864 0 0 nch w=1u l=180n
M6947 t2608 nw865 vdd vdd pch w=2u l=180n
M6948 t2608 t2607 vdd vdd pch w=2u l=180n
CT2611 t2611 0 0.1f
M6949 t2608 nw865 t2611 0 nch w=1u l=180n
M6950 t2611 t2607 0 0 nch w=1u l=180n
M6951 t2609 nw864 vdd vdd pch w=2u l=180n
M6952 t2609 t2607 vdd vdd pch w=2u l=180n
CT2612 t2612 0 0.1f
M6953 t2609 nw864 t2612 0 nch w=1u l=180n
M6954 t2612 t2607 0 0 nch w=1u l=180n
M6955 nw866 t2608 vdd vdd pch w=2u l=180n
M6956 nw866 t2609 vdd vdd pch w=2u l=180n
CT2613 t2613 0 0.1f
M6957 nw866 t2608 t2613 0 nch w=1u l=180n
M6958 t2613 t2609 0 0 nch w=1u l=180n
Cnw866 nw866 0 2f
M6959 nw867 nw144 vdd vdd pch w=2u l=180n
M6960 nw867 nw792 vdd vdd pch w=2u l=180n
CT2614 t2614 0 0.1f
M6961 nw867 nw144 t2614 0 nch w=1u l=180n
M6962 t2614 nw792 0 0 nch w=1u l=180n
Cnw867 nw867 0 2f
M6963 nw868 nw865 vdd vdd pch w=2u l=180n
M6964 nw868 nw864 vdd vdd pch w=2u l=180n
CT2615 t2615 0 0.1f
M6965 nw868 nw865 t2615 0 nch w=1u l=180n
M6966 t2615 nw864 0 0 nch w=1u l=180n
Cnw868 nw868 0 2f
M6967 nw869 nw867 vdd vdd pch w=2u l=180n
M6968 nw869 nw868 vdd vdd pch w=2u l=180n
CT2616 t2616 0 0.1f
M6969 nw869 nw867 t2616 0 nch w=1u l=180n
M6970 t2616 nw868 0 0 nch w=1u l=180n
Cnw869 nw869 0 2f
CT2617 t2617 0 0.1f
CT2618 t2618 0 0.1f
CT2619 t2619 0 0.1f
M6971 t2617 nw145 vdd vdd pch w=2u l=180n
M6972 t2617 nw796 vdd vdd pch w=2u l=180n
CT2620 t2620 0 0.1f
M6973 t2617 nw145 t2620 0 nch w=1u l=180n
M6974 t2620 nw796 0 0 nch w=1u l=180n
M6975 t2618 nw145 vdd vdd pch w=2u l=180n
M6976 t2618 t2617 vdd vdd pch w=2u l=180n
CT2621 t2621 0 0.1f
M6977 t2618 nw145 t2621 0 nch w=1u l=180n
M6978 t2621 t2617 0 0 nch w=1u l=180n
M6979 t2619 nw796 vdd vdd pch w=2u l=180n
M6980 t2619 t2617 vdd vdd pch w=2u l=180n
CT2622 t2622 0 0.1f
M6981 t2619 nw796 t2622 0 nch w=1u l=180n
M6982 t2622 t2617 0 0 nch w=1u l=180n
M6983 nw870 t2618 vdd vdd pch w=2u l=180n
M6984 nw870 t2619 vdd vdd pch w=2u l=180n
CT2623 t2623 0 0.1f
M6985 nw870 t2618 t2623 0 nch w=1u l=180n
M6986 t2623 t2619 0 0 nch w=1u l=180n
Cnw870 nw870 0 2f
CT2624 t2624 0 0.1f
M6987 t2624 nw145 vdd vdd pch w=2u l=180n
M6988 t2624 nw796 vdd vdd pch w=2u l=180n
CT2625 t2625 0 0.1f
M6989 t2624 nw145 t2625 0 nch w=1u l=180n
M6990 t2625 nw796 0 0 nch w=1u l=180n
M6991 nw871 t2624 vdd vdd pch w=2u l=180n
M6992 nw871 t2624 0 0 nch w=1u l=180n
Cnw871 nw871 0 2f
CT2626 t2626 0 0.1f
CT2627 t2627 0 0.1f
CT2628 t2628 0 0.1f
M6993 t2626 nw146 vdd vdd pch w=2u l=180n
M6994 t2626 nw801 vdd vdd pch w=2u l=180n
CT2629 t2629 0 0.1f
M6995 t2626 nw146 t2629 0 nch w=1u l=180n
M6996 t2629 nw801 0 0 nch w=1u l=180n
M6997 t2627 nw146 vdd vdd pch w=2u l=180n
M6998 t2627 t2626 vdd vdd pch w=2u l=180n
CT2630 t2630 0 0.1f
M6999 t2627 nw146 t2630 0 nch w=1u l=180n
M7000 t2630 t2626 0 0 nch w=1u l=180n
M7001 t2628 nw801 vdd vdd pch w=2u l=180n
M7002 t2628 t2626 vdd vdd pch w=2u l=180n
CT2631 t2631 0 0.1f
M7003 t2628 nw801 t2631 0 nch w=1u l=180n
M7004 t2631 t2626 0 0 nch w=1u l=180n
M7005 nw872 t2627 vdd vdd pch w=2u l=180n
M7006 nw872 t2628 vdd vdd pch w=2u l=180n
CT2632 t2632 0 0.1f
M7007 nw872 t2627 t2632 0 nch w=1u l=180n
M7008 t2632 t2628 0 0 nch w=1u l=180n
Cnw872 nw872 0 2f
CT2633 t2633 0 0.1f
CT2634 t2634 0 0.1f
CT2635 t2635 0 0.1f
M7009 t2633 nw872 vdd vdd pch w=2u l=180n
M7010 t2633 nw871 vdd vdd pch w=2u l=180n
CT2636 t2636 0 0.1f
M7011 t2633 nw872 t2636 0 nch w=1u l=180n
M7012 t2636 nw871 0 0 nch w=1u l=180n
M7013 t2634 nw872 vdd vdd pch w=2u l=180n
M7014 t2634 t2633 vdd vdd pch w=2u l=180n
CT2637 t2637 0 0.1f
M7015 t2634 nw872 t2637 0 nch w=1u l=180n
M7016 t2637 t2633 0 0 nch w=1u l=180n
M7017 t2635 nw871 vdd vdd pch w=2u l=180n
M7018 t2635 t2633 vdd vdd pch w=2u l=180n
CT2638 t2638 0 0.1f
M7019 t2635 nw871 t2638 0 nch w=1u l=180n
M7020 t2638 t2633 0 0 nch w=1u l=180n
M7021 nw873 t2634 vdd vdd pch w=2u l=180n
M7022 nw873 t2635 vdd vdd pch w=2u l=180n
CT2639 t2639 0 0.1f
M7023 nw873 t2634 t2639 0 nch w=1u l=180n
M7024 t2639 t2635 0 0 nch w=1u l=180n
Cnw873 nw873 0 2f
M7025 nw874 nw146 vdd vdd pch w=2u l=180n
M7026 nw874 nw801 vdd vdd pch w=2u l=180n
CT2640 t2640 0 0.1f
M7027 nw874 nw146 t2640 0 nch w=1u l=180n
M7028 t2640 nw801 0 0 nch w=1u l=180n
Cnw874 nw874 0 2f
M7029 nw875 nw872 vdd vdd pch w=2u l=180n
M7030 nw875 nw871 vdd vdd pch w=2u l=180n
CT2641 t2641 0 0.1f
M7031 nw875 nw872 t2641 0 nch w=1u l=180n
M7032 t2641 nw871 0 0 nch w=1u l=180n
Cnw875 nw875 0 2f
M7033 nw876 nw874 vdd vdd pch w=2u l=180n
M7034 nw876 nw875 vdd vdd pch w=2u l=180n
CT2642 t2642 0 0.1f
M7035 nw876 nw874 t2642 0 nch w=1u l=180n
M7036 t2642 nw875 0 0 nch w=1u l=180n
Cnw876 nw876 0 2f
CT2643 t2643 0 0.1f
CT2644 t2644 0 0.1f
CT2645 t2645 0 0.1f
M7037 t2643 nw147 vdd vdd pch w=2u l=180n
M7038 t2643 nw806 vdd vdd pch w=2u l=180n
CT2646 t2646 0 0.1f
M7039 t2643 nw147 t2646 0 nch w=1u l=180n
M7040 t2646 nw806 0 0 nch w=1u l=180n
M7041 t2644 nw147 vdd vdd pch w=2u l=180n
M7042 t2644 t2643 vdd vdd pch w=2u l=180n
CT2647 t2647 0 0.1f
M7043 t2644 nw147 t2647 0 nch w=1u l=180n
M7044 t2647 t2643 0 0 nch w=1u l=180n
M7045 t2645 nw806 vdd vdd pch w=2u l=180n
M7046 t2645 t2643 vdd vdd pch w=2u l=180n
CT2648 t2648 0 0.1f
M7047 t2645 nw806 t2648 0 nch w=1u l=180n
M7048 t2648 t2643 0 0 nch w=1u l=180n
M7049 nw877 t2644 vdd vdd pch w=2u l=180n
M7050 nw877 t2645 vdd vdd pch w=2u l=180n
CT2649 t2649 0 0.1f
M7051 nw877 t2644 t2649 0 nch w=1u l=180n
M7052 t2649 t2645 0 0 nch w=1u l=180n
Cnw877 nw877 0 2f
CT2650 t2650 0 0.1f
CT2651 t2651 0 0.1f
CT2652 t2652 0 0.1f
M7053 t2650 nw877 vdd vdd pch w=2u l=180n
M7054 t2650 nw876 vdd vdd pch w=2u l=180n
CT2653 t2653 0 0.1f
M7055 t2650 nw877 t2653 0 nch w=1u l=180n
M7056 t2653 nw876 0 0 nch w=1u l=180n
M7057 t2651 nw877 vdd vdd pch w=2u l=180n
M7058 t2651 t2650 vdd vdd pch w=2u l=180n
CT2654 t2654 0 0.1f
M7059 t2651 nw877 t2654 0 nch w=1u l=180n
M7060 t2654 t2650 0 0 nch w=1u l=180n
M7061 t2652 nw876 vdd vdd pch w=2u l=180n
M7062 t2652 t2650 vdd vdd pch w=2u l=180n
CT2655 t2655 0 0.1f
M7063 t2652 nw876 t2655 0 nch w=1u l=180n
M7064 t2655 t2650 0 0 nch w=1u l=180n
M7065 nw878 t2651 vdd vdd pch w=2u l=180n
M7066 nw878 t2652 vdd vdd pch w=2u l=180n
CT2656 t2656 0 0.1f
M7067 nw878 t2651 t2656 0 nch w=1u l=180n
M7068 t2656 t2652 0 0 nch w=1u l=180n
Cnw878 nw878 0 2f
M7069 nw879 nw147 vdd vdd pch w=2u l=180n
M7070 nw879 nw806 vdd vdd pch w=2u l=180n
CT2657 t2657 0 0.1f
M7071 nw879 nw147 t2657 0 nch w=1u l=180n
M7072 t2657 nw806 0 0 nch w=1u l=180n
Cnw879 nw879 0 2f
M7073 nw880 nw877 vdd vdd pch w=2u l=180n
M7074 nw880 nw876 vdd vdd pch w=2u l=180n
CT2658 t2658 0 0.1f
M7075 nw880 nw877 t2658 0 nch w=1u l=180n
M7076 t2658 nw876 0 0 nch w=1u l=180n
Cnw880 nw880 0 2f
M7077 nw881 nw879 vdd vdd pch w=2u l=180n
M7078 nw881 nw880 vdd vdd pch w=2u l=180n
CT2659 t2659 0 0.1f
M7079 nw881 nw879 t2659 0 nch w=1u l=180n
M7080 t2659 nw880 0 0 nch w=1u l=180n
Cnw881 nw881 0 2f
CT2660 t2660 0 0.1f
CT2661 t2661 0 0.1f
CT2662 t2662 0 0.1f
M7081 t2660 nw148 vdd vdd pch w=2u l=180n
M7082 t2660 nw811 vdd vdd pch w=2u l=180n
CT2663 t2663 0 0.1f
M7083 t2660 nw148 t2663 0 nch w=1u l=180n
M7084 t2663 nw811 0 0 nch w=1u l=180n
M7085 t2661 nw148 vdd vdd pch w=2u l=180n
M7086 t2661 t2660 vdd vdd pch w=2u l=180n
CT2664 t2664 0 0.1f
M7087 t2661 nw148 t2664 0 nch w=1u l=180n
M7088 t2664 t2660 0 0 nch w=1u l=180n
M7089 t2662 nw811 vdd vdd pch w=2u l=180n
M7090 t2662 t2660 vdd vdd pch w=2u l=180n
CT2665 t2665 0 0.1f
M7091 t2662 nw811 t2665 0 nch w=1u l=180n
M7092 t2665 t2660 0 0 nch w=1u l=180n
M7093 nw882 t2661 vdd vdd pch w=2u l=180n
M7094 nw882 t2662 vdd vdd pch w=2u l=180n
CT2666 t2666 0 0.1f
M7095 nw882 t2661 t2666 0 nch w=1u l=180n
M7096 t2666 t2662 0 0 nch w=1u l=180n
Cnw882 nw882 0 2f
CT2667 t2667 0 0.1f
CT2668 t2668 0 0.1f
CT2669 t2669 0 0.1f
M7097 t2667 nw882 vdd vdd pch w=2u l=180n
M7098 t2667 nw881 vdd vdd pch w=2u l=180n
CT2670 t2670 0 0.1f
M7099 t2667 nw882 t2670 0 nch w=1u l=180n
M7100 t2670 nw881 0 0 nch w=1u l=180n
M7101 t2668 nw882 vdd vdd pch w=2u l=180n
M7102 t2668 t2667 vdd vdd pch w=2u l=180n
CT2671 t2671 0 0.1f
M7103 t2668 nw882 t2671 0 nch w=1u l=180n
M7104 t2671 t2667 0 0 nch w=1u l=180n
M7105 t2669 nw881 vdd vdd pch w=2u l=180n
M7106 t2669 t2667 vdd vdd pch w=2u l=180n
CT2672 t2672 0 0.1f
M7107 t2669 nw881 t2672 0 nch w=1u l=180n
M7108 t2672 t2667 0 0 nch w=1u l=180n
M7109 nw883 t2668 vdd vdd pch w=2u l=180n
M7110 nw883 t2669 vdd vdd pch w=2u l=180n
CT2673 t2673 0 0.1f
M7111 nw883 t2668 t2673 0 nch w=1u l=180n
M7112 t2673 t2669 0 0 nch w=1u l=180n
Cnw883 nw883 0 2f
M7113 nw884 nw148 vdd vdd pch w=2u l=180n
M7114 nw884 nw811 vdd vdd pch w=2u l=180n
CT2674 t2674 0 0.1f
M7115 nw884 nw148 t2674 0 nch w=1u l=180n
M7116 t2674 nw811 0 0 nch w=1u l=180n
Cnw884 nw884 0 2f
M7117 nw885 nw882 vdd vdd pch w=2u l=180n
M7118 nw885 nw881 vdd vdd pch w=2u l=180n
CT2675 t2675 0 0.1f
M7119 nw885 nw882 t2675 0 nch w=1u l=180n
M7120 t2675 nw881 0 0 nch w=1u l=180n
Cnw885 nw885 0 2f
M7121 nw886 nw884 vdd vdd pch w=2u l=180n
M7122 nw886 nw885 vdd vdd pch w=2u l=180n
CT2676 t2676 0 0.1f
M7123 nw886 nw884 t2676 0 nch w=1u l=180n
M7124 t2676 nw885 0 0 nch w=1u l=180n
Cnw886 nw886 0 2f
CT2677 t2677 0 0.1f
CT2678 t2678 0 0.1f
CT2679 t2679 0 0.1f
M7125 t2677 nw149 vdd vdd pch w=2u l=180n
M7126 t2677 nw816 vdd vdd pch w=2u l=180n
CT2680 t2680 0 0.1f
M7127 t2677 nw149 t2680 0 nch w=1u l=180n
M7128 t2680 nw816 0 0 nch w=1u l=180n
M7129 t2678 nw149 vdd vdd pch w=2u l=180n
M7130 t2678 t2677 vdd vdd pch w=2u l=180n
CT2681 t2681 0 0.1f
M7131 t2678 nw149 t2681 0 nch w=1u l=180n
M7132 t2681 t2677 0 0 nch w=1u l=180n
M7133 t2679 nw816 vdd vdd pch w=2u l=180n
M7134 t2679 t2677 vdd vdd pch w=2u l=180n
CT2682 t2682 0 0.1f
M7135 t2679 nw816 t2682 0 nch w=1u l=180n
M7136 t2682 t2677 0 0 nch w=1u l=180n
M7137 nw887 t2678 vdd vdd pch w=2u l=180n
M7138 nw887 t2679 vdd vdd pch w=2u l=180n
CT2683 t2683 0 0.1f
M7139 nw887 t2678 t2683 0 nch w=1u l=180n
M7140 t2683 t2679 0 0 nch w=1u l=180n
Cnw887 nw887 0 2f
CT2684 t2684 0 0.1f
CT2685 t2685 0 0.1f
CT2686 t2686 0 0.1f
M7141 t2684 nw887 vdd vdd pch w=2u l=180n
M7142 t2684 nw886 vdd vdd pch w=2u l=180n
CT2687 t2687 0 0.1f
M7143 t2684 nw887 t2687 0 nch w=1u l=180n
M7144 t2687 nw886 0 0 nch w=1u l=180n
M7145 t2685 nw887 vdd vdd pch w=2u l=180n
M7146 t2685 t2684 vdd vdd pch w=2u l=180n
CT2688 t2688 0 0.1f
M7147 t2685 nw887 t2688 0 nch w=1u l=180n
M7148 t2688 t2684 0 0 nch w=1u l=180n
M7149 t2686 nw886 vdd vdd pch w=2u l=180n
M7150 t2686 t2684 vdd vdd pch w=2u l=180n
CT2689 t2689 0 0.1f
M7151 t2686 nw886 t2689 0 nch w=1u l=180n
M7152 t2689 t2684 0 0 nch w=1u l=180n
M7153 nw888 t2685 vdd vdd pch w=2u l=180n
M7154 nw888 t2686 vdd vdd pch w=2u l=180n
CT2690 t2690 0 0.1f
M7155 nw888 t2685 t2690 0 nch w=1u l=180n
M7156 t2690 t2686 0 0 nch w=1u l=180n
Cnw888 nw888 0 2f
M7157 nw889 nw149 vdd vdd pch w=2u l=180n
M7158 nw889 nw816 vdd vdd pch w=2u l=180n
CT2691 t2691 0 0.1f
M7159 nw889 nw149 t2691 0 nch w=1u l=180n
M7160 t2691 nw816 0 0 nch w=1u l=180n
Cnw889 nw889 0 2f
M7161 nw890 nw887 vdd vdd pch w=2u l=180n
M7162 nw890 nw886 vdd vdd pch w=2u l=180n
CT2692 t2692 0 0.1f
M7163 nw890 nw887 t2692 0 nch w=1u l=180n
M7164 t2692 nw886 0 0 nch w=1u l=180n
Cnw890 nw890 0 2f
M7165 nw891 nw889 vdd vdd pch w=2u l=180n
M7166 nw891 nw890 vdd vdd pch w=2u l=180n
CT2693 t2693 0 0.1f
M7167 nw891 nw889 t2693 0 nch w=1u l=180n
M7168 t2693 nw890 0 0 nch w=1u l=180n
Cnw891 nw891 0 2f
CT2694 t2694 0 0.1f
CT2695 t2695 0 0.1f
CT2696 t2696 0 0.1f
M7169 t2694 nw150 vdd vdd pch w=2u l=180n
M7170 t2694 nw821 vdd vdd pch w=2u l=180n
CT2697 t2697 0 0.1f
M7171 t2694 nw150 t2697 0 nch w=1u l=180n
M7172 t2697 nw821 0 0 nch w=1u l=180n
M7173 t2695 nw150 vdd vdd pch w=2u l=180n
M7174 t2695 t2694 vdd vdd pch w=2u l=180n
CT2698 t2698 0 0.1f
M7175 t2695 nw150 t2698 0 nch w=1u l=180n
M7176 t2698 t2694 0 0 nch w=1u l=180n
M7177 t2696 nw821 vdd vdd pch w=2u l=180n
M7178 t2696 t2694 vdd vdd pch w=2u l=180n
CT2699 t2699 0 0.1f
M7179 t2696 nw821 t2699 0 nch w=1u l=180n
M7180 t2699 t2694 0 0 nch w=1u l=180n
M7181 nw892 t2695 vdd vdd pch w=2u l=180n
M7182 nw892 t2696 vdd vdd pch w=2u l=180n
CT2700 t2700 0 0.1f
M7183 nw892 t2695 t2700 0 nch w=1u l=180n
M7184 t2700 t2696 0 0 nch w=1u l=180n
Cnw892 nw892 0 2f
CT2701 t2701 0 0.1f
CT2702 t2702 0 0.1f
CT2703 t2703 0 0.1f
M7185 t2701 nw892 vdd vdd pch w=2u l=180n
M7186 t2701 nw891 vdd vdd pch w=2u l=180n
CT2704 t2704 0 0.1f
M7187 t2701 nw892 t2704 0 nch w=1u l=180n
M7188 t2704 nw891 0 0 nch w=1u l=180n
M7189 t2702 nw892 vdd vdd pch w=2u l=180n
M7190 t2702 t2701 vdd vdd pch w=2u l=180n
CT2705 t2705 0 0.1f
M7191 t2702 nw892 t2705 0 nch w=1u l=180n
M7192 t2705 t2701 0 0 nch w=1u l=180n
M7193 t2703 nw891 vdd vdd pch w=2u l=180n
M7194 t2703 t2701 vdd vdd pch w=2u l=180n
CT2706 t2706 0 0.1f
M7195 t2703 nw891 t2706 0 nch w=1u l=180n
M7196 t2706 t2701 0 0 nch w=1u l=180n
M7197 nw893 t2702 vdd vdd pch w=2u l=180n
M7198 nw893 t2703 vdd vdd pch w=2u l=180n
CT2707 t2707 0 0.1f
M7199 nw893 t2702 t2707 0 nch w=1u l=180n
M7200 t2707 t2703 0 0 nch w=1u l=180n
Cnw893 nw893 0 2f
M7201 nw894 nw150 vdd vdd pch w=2u l=180n
M7202 nw894 nw821 vdd vdd pch w=2u l=180n
CT2708 t2708 0 0.1f
M7203 nw894 nw150 t2708 0 nch w=1u l=180n
M7204 t2708 nw821 0 0 nch w=1u l=180n
Cnw894 nw894 0 2f
M7205 nw895 nw892 vdd vdd pch w=2u l=180n
M7206 nw895 nw891 vdd vdd pch w=2u l=180n
CT2709 t2709 0 0.1f
M7207 nw895 nw892 t2709 0 nch w=1u l=180n
M7208 t2709 nw891 0 0 nch w=1u l=180n
Cnw895 nw895 0 2f
M7209 nw896 nw894 vdd vdd pch w=2u l=180n
M7210 nw896 nw895 vdd vdd pch w=2u l=180n
CT2710 t2710 0 0.1f
M7211 nw896 nw894 t2710 0 nch w=1u l=180n
M7212 t2710 nw895 0 0 nch w=1u l=180n
Cnw896 nw896 0 2f
CT2711 t2711 0 0.1f
CT2712 t2712 0 0.1f
CT2713 t2713 0 0.1f
M7213 t2711 nw151 vdd vdd pch w=2u l=180n
M7214 t2711 nw826 vdd vdd pch w=2u l=180n
CT2714 t2714 0 0.1f
M7215 t2711 nw151 t2714 0 nch w=1u l=180n
M7216 t2714 nw826 0 0 nch w=1u l=180n
M7217 t2712 nw151 vdd vdd pch w=2u l=180n
M7218 t2712 t2711 vdd vdd pch w=2u l=180n
CT2715 t2715 0 0.1f
M7219 t2712 nw151 t2715 0 nch w=1u l=180n
M7220 t2715 t2711 0 0 nch w=1u l=180n
M7221 t2713 nw826 vdd vdd pch w=2u l=180n
M7222 t2713 t2711 vdd vdd pch w=2u l=180n
CT2716 t2716 0 0.1f
M7223 t2713 nw826 t2716 0 nch w=1u l=180n
M7224 t2716 t2711 0 0 nch w=1u l=180n
M7225 nw897 t2712 vdd vdd pch w=2u l=180n
M7226 nw897 t2713 vdd vdd pch w=2u l=180n
CT2717 t2717 0 0.1f
M7227 nw897 t2712 t2717 0 nch w=1u l=180n
M7228 t2717 t2713 0 0 nch w=1u l=180n
Cnw897 nw897 0 2f
CT2718 t2718 0 0.1f
CT2719 t2719 0 0.1f
CT2720 t2720 0 0.1f
M7229 t2718 nw897 vdd vdd pch w=2u l=180n
M7230 t2718 nw896 vdd vdd pch w=2u l=180n
CT2721 t2721 0 0.1f
M7231 t2718 nw897 t2721 0 nch w=1u l=180n
M7232 t2721 nw896 0 0 nch w=1u l=180n
M7233 t2719 nw897 vdd vdd pch w=2u l=180n
M7234 t2719 t2718 vdd vdd pch w=2u l=180n
CT2722 t2722 0 0.1f
M7235 t2719 nw897 t2722 0 nch w=1u l=180n
M7236 t2722 t2718 0 0 nch w=1u l=180n
M7237 t2720 nw896 vdd vdd pch w=2u l=180n
M7238 t2720 t2718 vdd vdd pch w=2u l=180n
CT2723 t2723 0 0.1f
M7239 t2720 nw896 t2723 0 nch w=1u l=180n
M7240 t2723 t2718 0 0 nch w=1u l=180n
M7241 nw898 t2719 vdd vdd pch w=2u l=180n
M7242 nw898 t2720 vdd vdd pch w=2u l=180n
CT2724 t2724 0 0.1f
M7243 nw898 t2719 t2724 0 nch w=1u l=180n
M7244 t2724 t2720 0 0 nch w=1u l=180n
Cnw898 nw898 0 2f
M7245 nw899 nw151 vdd vdd pch w=2u l=180n
M7246 nw899 nw826 vdd vdd pch w=2u l=180n
CT2725 t2725 0 0.1f
M7247 nw899 nw151 t2725 0 nch w=1u l=180n
M7248 t2725 nw826 0 0 nch w=1u l=180n
Cnw899 nw899 0 2f
M7249 nw900 nw897 vdd vdd pch w=2u l=180n
M7250 nw900 nw896 vdd vdd pch w=2u l=180n
CT2726 t2726 0 0.1f
M7251 nw900 nw897 t2726 0 nch w=1u l=180n
M7252 t2726 nw896 0 0 nch w=1u l=180n
Cnw900 nw900 0 2f
M7253 nw901 nw899 vdd vdd pch w=2u l=180n
M7254 nw901 nw900 vdd vdd pch w=2u l=180n
CT2727 t2727 0 0.1f
M7255 nw901 nw899 t2727 0 nch w=1u l=180n
M7256 t2727 nw900 0 0 nch w=1u l=180n
Cnw901 nw901 0 2f
CT2728 t2728 0 0.1f
CT2729 t2729 0 0.1f
CT2730 t2730 0 0.1f
M7257 t2728 nw152 vdd vdd pch w=2u l=180n
M7258 t2728 nw831 vdd vdd pch w=2u l=180n
CT2731 t2731 0 0.1f
M7259 t2728 nw152 t2731 0 nch w=1u l=180n
M7260 t2731 nw831 0 0 nch w=1u l=180n
M7261 t2729 nw152 vdd vdd pch w=2u l=180n
M7262 t2729 t2728 vdd vdd pch w=2u l=180n
CT2732 t2732 0 0.1f
M7263 t2729 nw152 t2732 0 nch w=1u l=180n
M7264 t2732 t2728 0 0 nch w=1u l=180n
M7265 t2730 nw831 vdd vdd pch w=2u l=180n
M7266 t2730 t2728 vdd vdd pch w=2u l=180n
CT2733 t2733 0 0.1f
M7267 t2730 nw831 t2733 0 nch w=1u l=180n
M7268 t2733 t2728 0 0 nch w=1u l=180n
M7269 nw902 t2729 vdd vdd pch w=2u l=180n
M7270 nw902 t2730 vdd vdd pch w=2u l=180n
CT2734 t2734 0 0.1f
M7271 nw902 t2729 t2734 0 nch w=1u l=180n
M7272 t2734 t2730 0 0 nch w=1u l=180n
Cnw902 nw902 0 2f
CT2735 t2735 0 0.1f
CT2736 t2736 0 0.1f
CT2737 t2737 0 0.1f
M7273 t2735 nw902 vdd vdd pch w=2u l=180n
M7274 t2735 nw901 vdd vdd pch w=2u l=180n
CT2738 t2738 0 0.1f
M7275 t2735 nw902 t2738 0 nch w=1u l=180n
M7276 t2738 nw901 0 0 nch w=1u l=180n
M7277 t2736 nw902 vdd vdd pch w=2u l=180n
M7278 t2736 t2735 vdd vdd pch w=2u l=180n
CT2739 t2739 0 0.1f
M7279 t2736 nw902 t2739 0 nch w=1u l=180n
M7280 t2739 t2735 0 0 nch w=1u l=180n
M7281 t2737 nw901 vdd vdd pch w=2u l=180n
M7282 t2737 t2735 vdd vdd pch w=2u l=180n
CT2740 t2740 0 0.1f
M7283 t2737 nw901 t2740 0 nch w=1u l=180n
M7284 t2740 t2735 0 0 nch w=1u l=180n
M7285 nw903 t2736 vdd vdd pch w=2u l=180n
M7286 nw903 t2737 vdd vdd pch w=2u l=180n
CT2741 t2741 0 0.1f
M7287 nw903 t2736 t2741 0 nch w=1u l=180n
M7288 t2741 t2737 0 0 nch w=1u l=180n
Cnw903 nw903 0 2f
M7289 nw904 nw152 vdd vdd pch w=2u l=180n
M7290 nw904 nw831 vdd vdd pch w=2u l=180n
CT2742 t2742 0 0.1f
M7291 nw904 nw152 t2742 0 nch w=1u l=180n
M7292 t2742 nw831 0 0 nch w=1u l=180n
Cnw904 nw904 0 2f
M7293 nw905 nw902 vdd vdd pch w=2u l=180n
M7294 nw905 nw901 vdd vdd pch w=2u l=180n
CT2743 t2743 0 0.1f
M7295 nw905 nw902 t2743 0 nch w=1u l=180n
M7296 t2743 nw901 0 0 nch w=1u l=180n
Cnw905 nw905 0 2f
M7297 nw906 nw904 vdd vdd pch w=2u l=180n
M7298 nw906 nw905 vdd vdd pch w=2u l=180n
CT2744 t2744 0 0.1f
M7299 nw906 nw904 t2744 0 nch w=1u l=180n
M7300 t2744 nw905 0 0 nch w=1u l=180n
Cnw906 nw906 0 2f
CT2745 t2745 0 0.1f
CT2746 t2746 0 0.1f
CT2747 t2747 0 0.1f
M7301 t2745 nw153 vdd vdd pch w=2u l=180n
M7302 t2745 nw836 vdd vdd pch w=2u l=180n
CT2748 t2748 0 0.1f
M7303 t2745 nw153 t2748 0 nch w=1u l=180n
M7304 t2748 nw836 0 0 nch w=1u l=180n
M7305 t2746 nw153 vdd vdd pch w=2u l=180n
M7306 t2746 t2745 vdd vdd pch w=2u l=180n
CT2749 t2749 0 0.1f
M7307 t2746 nw153 t2749 0 nch w=1u l=180n
M7308 t2749 t2745 0 0 nch w=1u l=180n
M7309 t2747 nw836 vdd vdd pch w=2u l=180n
M7310 t2747 t2745 vdd vdd pch w=2u l=180n
CT2750 t2750 0 0.1f
M7311 t2747 nw836 t2750 0 nch w=1u l=180n
M7312 t2750 t2745 0 0 nch w=1u l=180n
M7313 nw907 t2746 vdd vdd pch w=2u l=180n
M7314 nw907 t2747 vdd vdd pch w=2u l=180n
CT2751 t2751 0 0.1f
M7315 nw907 t2746 t2751 0 nch w=1u l=180n
M7316 t2751 t2747 0 0 nch w=1u l=180n
Cnw907 nw907 0 2f
CT2752 t2752 0 0.1f
CT2753 t2753 0 0.1f
CT2754 t2754 0 0.1f
M7317 t2752 nw907 vdd vdd pch w=2u l=180n
M7318 t2752 nw906 vdd vdd pch w=2u l=180n
CT2755 t2755 0 0.1f
M7319 t2752 nw907 t2755 0 nch w=1u l=180n
M7320 t2755 nw906 0 0 nch w=1u l=180n
M7321 t2753 nw907 vdd vdd pch w=2u l=180n
M7322 t2753 t2752 vdd vdd pch w=2u l=180n
CT2756 t2756 0 0.1f
M7323 t2753 nw907 t2756 0 nch w=1u l=180n
M7324 t2756 t2752 0 0 nch w=1u l=180n
M7325 t2754 nw906 vdd vdd pch w=2u l=180n
M7326 t2754 t2752 vdd vdd pch w=2u l=180n
CT2757 t2757 0 0.1f
M7327 t2754 nw906 t2757 0 nch w=1u l=180n
M7328 t2757 t2752 0 0 nch w=1u l=180n
M7329 nw908 t2753 vdd vdd pch w=2u l=180n
M7330 nw908 t2754 vdd vdd pch w=2u l=180n
CT2758 t2758 0 0.1f
M7331 nw908 t2753 t2758 0 nch w=1u l=180n
M7332 t2758 t2754 0 0 nch w=1u l=180n
Cnw908 nw908 0 2f
M7333 nw909 nw153 vdd vdd pch w=2u l=180n
M7334 nw909 nw836 vdd vdd pch w=2u l=180n
CT2759 t2759 0 0.1f
M7335 nw909 nw153 t2759 0 nch w=1u l=180n
M7336 t2759 nw836 0 0 nch w=1u l=180n
Cnw909 nw909 0 2f
M7337 nw910 nw907 vdd vdd pch w=2u l=180n
M7338 nw910 nw906 vdd vdd pch w=2u l=180n
CT2760 t2760 0 0.1f
M7339 nw910 nw907 t2760 0 nch w=1u l=180n
M7340 t2760 nw906 0 0 nch w=1u l=180n
Cnw910 nw910 0 2f
M7341 nw911 nw909 vdd vdd pch w=2u l=180n
M7342 nw911 nw910 vdd vdd pch w=2u l=180n
CT2761 t2761 0 0.1f
M7343 nw911 nw909 t2761 0 nch w=1u l=180n
M7344 t2761 nw910 0 0 nch w=1u l=180n
Cnw911 nw911 0 2f
CT2762 t2762 0 0.1f
CT2763 t2763 0 0.1f
CT2764 t2764 0 0.1f
M7345 t2762 nw154 vdd vdd pch w=2u l=180n
M7346 t2762 nw841 vdd vdd pch w=2u l=180n
CT2765 t2765 0 0.1f
M7347 t2762 nw154 t2765 0 nch w=1u l=180n
M7348 t2765 nw841 0 0 nch w=1u l=180n
M7349 t2763 nw154 vdd vdd pch w=2u l=180n
M7350 t2763 t2762 vdd vdd pch w=2u l=180n
CT2766 t2766 0 0.1f
M7351 t2763 nw154 t2766 0 nch w=1u l=180n
M7352 t2766 t2762 0 0 nch w=1u l=180n
M7353 t2764 nw841 vdd vdd pch w=2u l=180n
M7354 t2764 t2762 vdd vdd pch w=2u l=180n
CT2767 t2767 0 0.1f
M7355 t2764 nw841 t2767 0 nch w=1u l=180n
M7356 t2767 t2762 0 0 nch w=1u l=180n
M7357 nw912 t2763 vdd vdd pch w=2u l=180n
M7358 nw912 t2764 vdd vdd pch w=2u l=180n
CT2768 t2768 0 0.1f
M7359 nw912 t2763 t2768 0 nch w=1u l=180n
M7360 t2768 t2764 0 0 nch w=1u l=180n
Cnw912 nw912 0 2f
CT2769 t2769 0 0.1f
CT2770 t2770 0 0.1f
CT2771 t2771 0 0.1f
M7361 t2769 nw912 vdd vdd pch w=2u l=180n
M7362 t2769 nw911 vdd vdd pch w=2u l=180n
CT2772 t2772 0 0.1f
M7363 t2769 nw912 t2772 0 nch w=1u l=180n
M7364 t2772 nw911 0 0 nch w=1u l=180n
M7365 t2770 nw912 vdd vdd pch w=2u l=180n
M7366 t2770 t2769 vdd vdd pch w=2u l=180n
CT2773 t2773 0 0.1f
M7367 t2770 nw912 t2773 0 nch w=1u l=180n
M7368 t2773 t2769 0 0 nch w=1u l=180n
M7369 t2771 nw911 vdd vdd pch w=2u l=180n
M7370 t2771 t2769 vdd vdd pch w=2u l=180n
CT2774 t2774 0 0.1f
M7371 t2771 nw911 t2774 0 nch w=1u l=180n
M7372 t2774 t2769 0 0 nch w=1u l=180n
M7373 nw913 t2770 vdd vdd pch w=2u l=180n
M7374 nw913 t2771 vdd vdd pch w=2u l=180n
CT2775 t2775 0 0.1f
M7375 nw913 t2770 t2775 0 nch w=1u l=180n
M7376 t2775 t2771 0 0 nch w=1u l=180n
Cnw913 nw913 0 2f
M7377 nw914 nw154 vdd vdd pch w=2u l=180n
M7378 nw914 nw841 vdd vdd pch w=2u l=180n
CT2776 t2776 0 0.1f
M7379 nw914 nw154 t2776 0 nch w=1u l=180n
M7380 t2776 nw841 0 0 nch w=1u l=180n
Cnw914 nw914 0 2f
M7381 nw915 nw912 vdd vdd pch w=2u l=180n
M7382 nw915 nw911 vdd vdd pch w=2u l=180n
CT2777 t2777 0 0.1f
M7383 nw915 nw912 t2777 0 nch w=1u l=180n
M7384 t2777 nw911 0 0 nch w=1u l=180n
Cnw915 nw915 0 2f
M7385 nw916 nw914 vdd vdd pch w=2u l=180n
M7386 nw916 nw915 vdd vdd pch w=2u l=180n
CT2778 t2778 0 0.1f
M7387 nw916 nw914 t2778 0 nch w=1u l=180n
M7388 t2778 nw915 0 0 nch w=1u l=180n
Cnw916 nw916 0 2f
CT2779 t2779 0 0.1f
CT2780 t2780 0 0.1f
CT2781 t2781 0 0.1f
M7389 t2779 nw155 vdd vdd pch w=2u l=180n
M7390 t2779 nw846 vdd vdd pch w=2u l=180n
CT2782 t2782 0 0.1f
M7391 t2779 nw155 t2782 0 nch w=1u l=180n
M7392 t2782 nw846 0 0 nch w=1u l=180n
M7393 t2780 nw155 vdd vdd pch w=2u l=180n
M7394 t2780 t2779 vdd vdd pch w=2u l=180n
CT2783 t2783 0 0.1f
M7395 t2780 nw155 t2783 0 nch w=1u l=180n
M7396 t2783 t2779 0 0 nch w=1u l=180n
M7397 t2781 nw846 vdd vdd pch w=2u l=180n
M7398 t2781 t2779 vdd vdd pch w=2u l=180n
CT2784 t2784 0 0.1f
M7399 t2781 nw846 t2784 0 nch w=1u l=180n
M7400 t2784 t2779 0 0 nch w=1u l=180n
M7401 nw917 t2780 vdd vdd pch w=2u l=180n
M7402 nw917 t2781 vdd vdd pch w=2u l=180n
CT2785 t2785 0 0.1f
M7403 nw917 t2780 t2785 0 nch w=1u l=180n
M7404 t2785 t2781 0 0 nch w=1u l=180n
Cnw917 nw917 0 2f
CT2786 t2786 0 0.1f
CT2787 t2787 0 0.1f
CT2788 t2788 0 0.1f
M7405 t2786 nw917 vdd vdd pch w=2u l=180n
M7406 t2786 nw916 vdd vdd pch w=2u l=180n
CT2789 t2789 0 0.1f
M7407 t2786 nw917 t2789 0 nch w=1u l=180n
M7408 t2789 nw916 0 0 nch w=1u l=180n
M7409 t2787 nw917 vdd vdd pch w=2u l=180n
M7410 t2787 t2786 vdd vdd pch w=2u l=180n
CT2790 t2790 0 0.1f
M7411 t2787 nw917 t2790 0 nch w=1u l=180n
M7412 t2790 t2786 0 0 nch w=1u l=180n
M7413 t2788 nw916 vdd vdd pch w=2u l=180n
M7414 t2788 t2786 vdd vdd pch w=2u l=180n
CT2791 t2791 0 0.1f
M7415 t2788 nw916 t2791 0 nch w=1u l=180n
M7416 t2791 t2786 0 0 nch w=1u l=180n
M7417 nw918 t2787 vdd vdd pch w=2u l=180n
M7418 nw918 t2788 vdd vdd pch w=2u l=180n
CT2792 t2792 0 0.1f
M7419 nw918 t2787 t2792 0 nch w=1u l=180n
M7420 t2792 t2788 0 0 nch w=1u l=180n
Cnw918 nw918 0 2f
M7421 nw919 nw155 vdd vdd pch w=2u l=180n
M7422 nw919 nw846 vdd vdd pch w=2u l=180n
CT2793 t2793 0 0.1f
M7423 nw919 nw155 t2793 0 nch w=1u l=180n
M7424 t2793 nw846 0 0 nch w=1u l=180n
Cnw919 nw919 0 2f
M7425 nw920 nw917 vdd vdd pch w=2u l=180n
M7426 nw920 nw916 vdd vdd pch w=2u l=180n
CT2794 t2794 0 0.1f
M7427 nw920 nw917 t2794 0 nch w=1u l=180n
M7428 t2794 nw916 0 0 nch w=1u l=180n
Cnw920 nw920 0 2f
M7429 nw921 nw919 vdd vdd pch w=2u l=180n
M7430 nw921 nw920 vdd vdd pch w=2u l=180n
CT2795 t2795 0 0.1f
M7431 nw921 nw919 t2795 0 nch w=1u l=180n
M7432 t2795 nw920 0 0 nch w=1u l=180n
Cnw921 nw921 0 2f
CT2796 t2796 0 0.1f
CT2797 t2797 0 0.1f
CT2798 t2798 0 0.1f
M7433 t2796 nw156 vdd vdd pch w=2u l=180n
M7434 t2796 nw851 vdd vdd pch w=2u l=180n
CT2799 t2799 0 0.1f
M7435 t2796 nw156 t2799 0 nch w=1u l=180n
M7436 t2799 nw851 0 0 nch w=1u l=180n
M7437 t2797 nw156 vdd vdd pch w=2u l=180n
M7438 t2797 t2796 vdd vdd pch w=2u l=180n
CT2800 t2800 0 0.1f
M7439 t2797 nw156 t2800 0 nch w=1u l=180n
M7440 t2800 t2796 0 0 nch w=1u l=180n
M7441 t2798 nw851 vdd vdd pch w=2u l=180n
M7442 t2798 t2796 vdd vdd pch w=2u l=180n
CT2801 t2801 0 0.1f
M7443 t2798 nw851 t2801 0 nch w=1u l=180n
M7444 t2801 t2796 0 0 nch w=1u l=180n
M7445 nw922 t2797 vdd vdd pch w=2u l=180n
M7446 nw922 t2798 vdd vdd pch w=2u l=180n
CT2802 t2802 0 0.1f
M7447 nw922 t2797 t2802 0 nch w=1u l=180n
M7448 t2802 t2798 0 0 nch w=1u l=180n
Cnw922 nw922 0 2f
CT2803 t2803 0 0.1f
CT2804 t2804 0 0.1f
CT2805 t2805 0 0.1f
M7449 t2803 nw922 vdd vdd pch w=2u l=180n
M7450 t2803 nw921 vdd vdd pch w=2u l=180n
CT2806 t2806 0 0.1f
M7451 t2803 nw922 t2806 0 nch w=1u l=180n
M7452 t2806 nw921 0 0 nch w=1u l=180n
M7453 t2804 nw922 vdd vdd pch w=2u l=180n
M7454 t2804 t2803 vdd vdd pch w=2u l=180n
CT2807 t2807 0 0.1f
M7455 t2804 nw922 t2807 0 nch w=1u l=180n
M7456 t2807 t2803 0 0 nch w=1u l=180n
M7457 t2805 nw921 vdd vdd pch w=2u l=180n
M7458 t2805 t2803 vdd vdd pch w=2u l=180n
CT2808 t2808 0 0.1f
M7459 t2805 nw921 t2808 0 nch w=1u l=180n
M7460 t2808 t2803 0 0 nch w=1u l=180n
M7461 nw923 t2804 vdd vdd pch w=2u l=180n
M7462 nw923 t2805 vdd vdd pch w=2u l=180n
CT2809 t2809 0 0.1f
M7463 nw923 t2804 t2809 0 nch w=1u l=180n
M7464 t2809 t2805 0 0 nch w=1u l=180n
Cnw923 nw923 0 2f
M7465 nw924 nw156 vdd vdd pch w=2u l=180n
M7466 nw924 nw851 vdd vdd pch w=2u l=180n
CT2810 t2810 0 0.1f
M7467 nw924 nw156 t2810 0 nch w=1u l=180n
M7468 t2810 nw851 0 0 nch w=1u l=180n
Cnw924 nw924 0 2f
M7469 nw925 nw922 vdd vdd pch w=2u l=180n
M7470 nw925 nw921 vdd vdd pch w=2u l=180n
CT2811 t2811 0 0.1f
M7471 nw925 nw922 t2811 0 nch w=1u l=180n
M7472 t2811 nw921 0 0 nch w=1u l=180n
Cnw925 nw925 0 2f
M7473 nw926 nw924 vdd vdd pch w=2u l=180n
M7474 nw926 nw925 vdd vdd pch w=2u l=180n
CT2812 t2812 0 0.1f
M7475 nw926 nw924 t2812 0 nch w=1u l=180n
M7476 t2812 nw925 0 0 nch w=1u l=180n
Cnw926 nw926 0 2f
CT2813 t2813 0 0.1f
CT2814 t2814 0 0.1f
CT2815 t2815 0 0.1f
M7477 t2813 nw157 vdd vdd pch w=2u l=180n
M7478 t2813 nw856 vdd vdd pch w=2u l=180n
CT2816 t2816 0 0.1f
M7479 t2813 nw157 t2816 0 nch w=1u l=180n
M7480 t2816 nw856 0 0 nch w=1u l=180n
M7481 t2814 nw157 vdd vdd pch w=2u l=180n
M7482 t2814 t2813 vdd vdd pch w=2u l=180n
CT2817 t2817 0 0.1f
M7483 t2814 nw157 t2817 0 nch w=1u l=180n
M7484 t2817 t2813 0 0 nch w=1u l=180n
M7485 t2815 nw856 vdd vdd pch w=2u l=180n
M7486 t2815 t2813 vdd vdd pch w=2u l=180n
CT2818 t2818 0 0.1f
M7487 t2815 nw856 t2818 0 nch w=1u l=180n
M7488 t2818 t2813 0 0 nch w=1u l=180n
M7489 nw927 t2814 vdd vdd pch w=2u l=180n
M7490 nw927 t2815 vdd vdd pch w=2u l=180n
CT2819 t2819 0 0.1f
M7491 nw927 t2814 t2819 0 nch w=1u l=180n
M7492 t2819 t2815 0 0 nch w=1u l=180n
Cnw927 nw927 0 2f
CT2820 t2820 0 0.1f
CT2821 t2821 0 0.1f
CT2822 t2822 0 0.1f
M7493 t2820 nw927 vdd vdd pch w=2u l=180n
M7494 t2820 nw926 vdd vdd pch w=2u l=180n
CT2823 t2823 0 0.1f
M7495 t2820 nw927 t2823 0 nch w=1u l=180n
M7496 t2823 nw926 0 0 nch w=1u l=180n
M7497 t2821 nw927 vdd vdd pch w=2u l=180n
M7498 t2821 t2820 vdd vdd pch w=2u l=180n
CT2824 t2824 0 0.1f
M7499 t2821 nw927 t2824 0 nch w=1u l=180n
M7500 t2824 t2820 0 0 nch w=1u l=180n
M7501 t2822 nw926 vdd vdd pch w=2u l=180n
M7502 t2822 t2820 vdd vdd pch w=2u l=180n
CT2825 t2825 0 0.1f
M7503 t2822 nw926 t2825 0 nch w=1u l=180n
M7504 t2825 t2820 0 0 nch w=1u l=180n
M7505 nw928 t2821 vdd vdd pch w=2u l=180n
M7506 nw928 t2822 vdd vdd pch w=2u l=180n
CT2826 t2826 0 0.1f
M7507 nw928 t2821 t2826 0 nch w=1u l=180n
M7508 t2826 t2822 0 0 nch w=1u l=180n
Cnw928 nw928 0 2f
M7509 nw929 nw157 vdd vdd pch w=2u l=180n
M7510 nw929 nw856 vdd vdd pch w=2u l=180n
CT2827 t2827 0 0.1f
M7511 nw929 nw157 t2827 0 nch w=1u l=180n
M7512 t2827 nw856 0 0 nch w=1u l=180n
Cnw929 nw929 0 2f
M7513 nw930 nw927 vdd vdd pch w=2u l=180n
M7514 nw930 nw926 vdd vdd pch w=2u l=180n
CT2828 t2828 0 0.1f
M7515 nw930 nw927 t2828 0 nch w=1u l=180n
M7516 t2828 nw926 0 0 nch w=1u l=180n
Cnw930 nw930 0 2f
M7517 nw931 nw929 vdd vdd pch w=2u l=180n
M7518 nw931 nw930 vdd vdd pch w=2u l=180n
CT2829 t2829 0 0.1f
M7519 nw931 nw929 t2829 0 nch w=1u l=180n
M7520 t2829 nw930 0 0 nch w=1u l=180n
Cnw931 nw931 0 2f
CT2830 t2830 0 0.1f
CT2831 t2831 0 0.1f
CT2832 t2832 0 0.1f
M7521 t2830 nw158 vdd vdd pch w=2u l=180n
M7522 t2830 nw861 vdd vdd pch w=2u l=180n
CT2833 t2833 0 0.1f
M7523 t2830 nw158 t2833 0 nch w=1u l=180n
M7524 t2833 nw861 0 0 nch w=1u l=180n
M7525 t2831 nw158 vdd vdd pch w=2u l=180n
M7526 t2831 t2830 vdd vdd pch w=2u l=180n
CT2834 t2834 0 0.1f
M7527 t2831 nw158 t2834 0 nch w=1u l=180n
M7528 t2834 t2830 0 0 nch w=1u l=180n
M7529 t2832 nw861 vdd vdd pch w=2u l=180n
M7530 t2832 t2830 vdd vdd pch w=2u l=180n
CT2835 t2835 0 0.1f
M7531 t2832 nw861 t2835 0 nch w=1u l=180n
M7532 t2835 t2830 0 0 nch w=1u l=180n
M7533 nw932 t2831 vdd vdd pch w=2u l=180n
M7534 nw932 t2832 vdd vdd pch w=2u l=180n
CT2836 t2836 0 0.1f
M7535 nw932 t2831 t2836 0 nch w=1u l=180n
M7536 t2836 t2832 0 0 nch w=1u l=180n
Cnw932 nw932 0 2f
CT2837 t2837 0 0.1f
CT2838 t2838 0 0.1f
CT2839 t2839 0 0.1f
M7537 t2837 nw932 vdd vdd pch w=2u l=180n
M7538 t2837 nw931 vdd vdd pch w=2u l=180n
CT2840 t2840 0 0.1f
M7539 t2837 nw932 t2840 0 nch w=1u l=180n
M7540 t2840 nw931 0 0 nch w=1u l=180n
M7541 t2838 nw932 vdd vdd pch w=2u l=180n
M7542 t2838 t2837 vdd vdd pch w=2u l=180n
CT2841 t2841 0 0.1f
M7543 t2838 nw932 t2841 0 nch w=1u l=180n
M7544 t2841 t2837 0 0 nch w=1u l=180n
M7545 t2839 nw931 vdd vdd pch w=2u l=180n
M7546 t2839 t2837 vdd vdd pch w=2u l=180n
CT2842 t2842 0 0.1f
M7547 t2839 nw931 t2842 0 nch w=1u l=180n
M7548 t2842 t2837 0 0 nch w=1u l=180n
M7549 nw933 t2838 vdd vdd pch w=2u l=180n
M7550 nw933 t2839 vdd vdd pch w=2u l=180n
CT2843 t2843 0 0.1f
M7551 nw933 t2838 t2843 0 nch w=1u l=180n
M7552 t2843 t2839 0 0 nch w=1u l=180n
Cnw933 nw933 0 2f
M7553 nw934 nw158 vdd vdd pch w=2u l=180n
M7554 nw934 nw861 vdd vdd pch w=2u l=180n
CT2844 t2844 0 0.1f
M7555 nw934 nw158 t2844 0 nch w=1u l=180n
M7556 t2844 nw861 0 0 nch w=1u l=180n
Cnw934 nw934 0 2f
M7557 nw935 nw932 vdd vdd pch w=2u l=180n
M7558 nw935 nw931 vdd vdd pch w=2u l=180n
CT2845 t2845 0 0.1f
M7559 nw935 nw932 t2845 0 nch w=1u l=180n
M7560 t2845 nw931 0 0 nch w=1u l=180n
Cnw935 nw935 0 2f
M7561 nw936 nw934 vdd vdd pch w=2u l=180n
M7562 nw936 nw935 vdd vdd pch w=2u l=180n
CT2846 t2846 0 0.1f
M7563 nw936 nw934 t2846 0 nch w=1u l=180n
M7564 t2846 nw935 0 0 nch w=1u l=180n
Cnw936 nw936 0 2f
CT2847 t2847 0 0.1f
CT2848 t2848 0 0.1f
CT2849 t2849 0 0.1f
M7565 t2847 nw159 vdd vdd pch w=2u l=180n
M7566 t2847 nw866 vdd vdd pch w=2u l=180n
CT2850 t2850 0 0.1f
M7567 t2847 nw159 t2850 0 nch w=1u l=180n
M7568 t2850 nw866 0 0 nch w=1u l=180n
M7569 t2848 nw159 vdd vdd pch w=2u l=180n
M7570 t2848 t2847 vdd vdd pch w=2u l=180n
CT2851 t2851 0 0.1f
M7571 t2848 nw159 t2851 0 nch w=1u l=180n
M7572 t2851 t2847 0 0 nch w=1u l=180n
M7573 t2849 nw866 vdd vdd pch w=2u l=180n
M7574 t2849 t2847 vdd vdd pch w=2u l=180n
CT2852 t2852 0 0.1f
M7575 t2849 nw866 t2852 0 nch w=1u l=180n
M7576 t2852 t2847 0 0 nch w=1u l=180n
M7577 nw937 t2848 vdd vdd pch w=2u l=180n
M7578 nw937 t2849 vdd vdd pch w=2u l=180n
CT2853 t2853 0 0.1f
M7579 nw937 t2848 t2853 0 nch w=1u l=180n
M7580 t2853 t2849 0 0 nch w=1u l=180n
Cnw937 nw937 0 2f
CT2854 t2854 0 0.1f
CT2855 t2855 0 0.1f
CT2856 t2856 0 0.1f
M7581 t2854 nw937 vdd vdd pch w=2u l=180n
M7582 t2854 nw936 vdd vdd pch w=2u l=180n
CT2857 t2857 0 0.1f
M7583 t2854 nw937 t2857 0 nch w=1u l=180n
M7584 t2857 nw936 0 0 nch w=1u l=180n
M7585 t2855 nw937 vdd vdd pch w=2u l=180n
M7586 t2855 t2854 vdd vdd pch w=2u l=180n
CT2858 t2858 0 0.1f
M7587 t2855 nw937 t2858 0 nch w=1u l=180n
M7588 t2858 t2854 0 0 nch w=1u l=180n
M7589 t2856 nw936 vdd vdd pch w=2u l=180n
M7590 t2856 t2854 vdd vdd pch w=2u l=180n
CT2859 t2859 0 0.1f
M7591 t2856 nw936 t2859 0 nch w=1u l=180n
M7592 t2859 t2854 0 0 nch w=1u l=180n
M7593 nw938 t2855 vdd vdd pch w=2u l=180n
M7594 nw938 t2856 vdd vdd pch w=2u l=180n
CT2860 t2860 0 0.1f
M7595 nw938 t2855 t2860 0 nch w=1u l=180n
M7596 t2860 t2856 0 0 nch w=1u l=180n
Cnw938 nw938 0 2f
M7597 nw939 nw159 vdd vdd pch w=2u l=180n
M7598 nw939 nw866 vdd vdd pch w=2u l=180n
CT2861 t2861 0 0.1f
M7599 nw939 nw159 t2861 0 nch w=1u l=180n
M7600 t2861 nw866 0 0 nch w=1u l=180n
Cnw939 nw939 0 2f
M7601 nw940 nw937 vdd vdd pch w=2u l=180n
M7602 nw940 nw936 vdd vdd pch w=2u l=180n
CT2862 t2862 0 0.1f
M7603 nw940 nw937 t2862 0 nch w=1u l=180n
M7604 t2862 nw936 0 0 nch w=1u l=180n
Cnw940 nw940 0 2f
M7605 nw941 nw939 vdd vdd pch w=2u l=180n
M7606 nw941 nw940 vdd vdd pch w=2u l=180n
CT2863 t2863 0 0.1f
M7607 nw941 nw939 t2863 0 nch w=1u l=180n
M7608 t2863 nw940 0 0 nch w=1u l=180n
Cnw941 nw941 0 2f
CT2864 t2864 0 0.1f
CT2865 t2865 0 0.1f
CT2866 t2866 0 0.1f
M7609 t2864 nw160 vdd vdd pch w=2u l=180n
M7610 t2864 nw869 vdd vdd pch w=2u l=180n
CT2867 t2867 0 0.1f
M7611 t2864 nw160 t2867 0 nch w=1u l=180n
M7612 t2867 nw869 0 0 nch w=1u l=180n
M7613 t2865 nw160 vdd vdd pch w=2u l=180n
M7614 t2865 t2864 vdd vdd pch w=2u l=180n
CT2868 t2868 0 0.1f
M7615 t2865 nw160 t2868 0 nch w=1u l=180n
M7616 t2868 t2864 0 0 nch w=1u l=180n
M7617 t2866 nw869 vdd vdd pch w=2u l=180n
M7618 t2866 t2864 vdd vdd pch w=2u l=180n
CT2869 t2869 0 0.1f
M7619 t2866 nw869 t2869 0 nch w=1u l=180n
M7620 t2869 t2864 0 0 nch w=1u l=180n
M7621 nw942 t2865 vdd vdd pch w=2u l=180n
M7622 nw942 t2866 vdd vdd pch w=2u l=180n
CT2870 t2870 0 0.1f
M7623 nw942 t2865 t2870 0 nch w=1u l=180n
M7624 t2870 t2866 0 0 nch w=1u l=180n
Cnw942 nw942 0 2f
CT2871 t2871 0 0.1f
CT2872 t2872 0 0.1f
CT2873 t2873 0 0.1f
M7625 t2871 nw942 vdd vdd pch w=2u l=180n
M7626 t2871 nw941 vdd vdd pch w=2u l=180n
CT2874 t2874 0 0.1f
M7627 t2871 nw942 t2874 0 nch w=1u l=180n
M7628 t2874 nw941 0 0 nch w=1u l=180n
M7629 t2872 nw942 vdd vdd pch w=2u l=180n
M7630 t2872 t2871 vdd vdd pch w=2u l=180n
CT2875 t2875 0 0.1f
M7631 t2872 nw942 t2875 0 nch w=1u l=180n
M7632 t2875 t2871 0 0 nch w=1u l=180n
M7633 t2873 nw941 vdd vdd pch w=2u l=180n
M7634 t2873 t2871 vdd vdd pch w=2u l=180n
CT2876 t2876 0 0.1f
M7635 t2873 nw941 t2876 0 nch w=1u l=180n
M7636 t2876 t2871 0 0 nch w=1u l=180n
M7637 nw943 t2872 vdd vdd pch w=2u l=180n
M7638 nw943 t2873 vdd vdd pch w=2u l=180n
CT2877 t2877 0 0.1f
M7639 nw943 t2872 t2877 0 nch w=1u l=180n
M7640 t2877 t2873 0 0 nch w=1u l=180n
Cnw943 nw943 0 2f
M7641 nw944 nw160 vdd vdd pch w=2u l=180n
M7642 nw944 nw869 vdd vdd pch w=2u l=180n
CT2878 t2878 0 0.1f
M7643 nw944 nw160 t2878 0 nch w=1u l=180n
M7644 t2878 nw869 0 0 nch w=1u l=180n
Cnw944 nw944 0 2f
M7645 nw945 nw942 vdd vdd pch w=2u l=180n
M7646 nw945 nw941 vdd vdd pch w=2u l=180n
CT2879 t2879 0 0.1f
M7647 nw945 nw942 t2879 0 nch w=1u l=180n
M7648 t2879 nw941 0 0 nch w=1u l=180n
Cnw945 nw945 0 2f
M7649 nw946 nw944 vdd vdd pch w=2u l=180n
M7650 nw946 nw945 vdd vdd pch w=2u l=180n
CT2880 t2880 0 0.1f
M7651 nw946 nw944 t2880 0 nch w=1u l=180n
M7652 t2880 nw945 0 0 nch w=1u l=180n
Cnw946 nw946 0 2f
CT2881 t2881 0 0.1f
CT2882 t2882 0 0.1f
CT2883 t2883 0 0.1f
M7653 t2881 nw161 vdd vdd pch w=2u l=180n
M7654 t2881 nw873 vdd vdd pch w=2u l=180n
CT2884 t2884 0 0.1f
M7655 t2881 nw161 t2884 0 nch w=1u l=180n
M7656 t2884 nw873 0 0 nch w=1u l=180n
M7657 t2882 nw161 vdd vdd pch w=2u l=180n
M7658 t2882 t2881 vdd vdd pch w=2u l=180n
CT2885 t2885 0 0.1f
M7659 t2882 nw161 t2885 0 nch w=1u l=180n
M7660 t2885 t2881 0 0 nch w=1u l=180n
M7661 t2883 nw873 vdd vdd pch w=2u l=180n
M7662 t2883 t2881 vdd vdd pch w=2u l=180n
CT2886 t2886 0 0.1f
M7663 t2883 nw873 t2886 0 nch w=1u l=180n
M7664 t2886 t2881 0 0 nch w=1u l=180n
M7665 nw947 t2882 vdd vdd pch w=2u l=180n
M7666 nw947 t2883 vdd vdd pch w=2u l=180n
CT2887 t2887 0 0.1f
M7667 nw947 t2882 t2887 0 nch w=1u l=180n
M7668 t2887 t2883 0 0 nch w=1u l=180n
Cnw947 nw947 0 2f
CT2888 t2888 0 0.1f
M7669 t2888 nw161 vdd vdd pch w=2u l=180n
M7670 t2888 nw873 vdd vdd pch w=2u l=180n
CT2889 t2889 0 0.1f
M7671 t2888 nw161 t2889 0 nch w=1u l=180n
M7672 t2889 nw873 0 0 nch w=1u l=180n
M7673 nw948 t2888 vdd vdd pch w=2u l=180n
M7674 nw948 t2888 0 0 nch w=1u l=180n
Cnw948 nw948 0 2f
CT2890 t2890 0 0.1f
CT2891 t2891 0 0.1f
CT2892 t2892 0 0.1f
M7675 t2890 nw162 vdd vdd pch w=2u l=180n
M7676 t2890 nw878 vdd vdd pch w=2u l=180n
CT2893 t2893 0 0.1f
M7677 t2890 nw162 t2893 0 nch w=1u l=180n
M7678 t2893 nw878 0 0 nch w=1u l=180n
M7679 t2891 nw162 vdd vdd pch w=2u l=180n
M7680 t2891 t2890 vdd vdd pch w=2u l=180n
CT2894 t2894 0 0.1f
M7681 t2891 nw162 t2894 0 nch w=1u l=180n
M7682 t2894 t2890 0 0 nch w=1u l=180n
M7683 t2892 nw878 vdd vdd pch w=2u l=180n
M7684 t2892 t2890 vdd vdd pch w=2u l=180n
CT2895 t2895 0 0.1f
M7685 t2892 nw878 t2895 0 nch w=1u l=180n
M7686 t2895 t2890 0 0 nch w=1u l=180n
M7687 nw949 t2891 vdd vdd pch w=2u l=180n
M7688 nw949 t2892 vdd vdd pch w=2u l=180n
CT2896 t2896 0 0.1f
M7689 nw949 t2891 t2896 0 nch w=1u l=180n
M7690 t2896 t2892 0 0 nch w=1u l=180n
Cnw949 nw949 0 2f
CT2897 t2897 0 0.1f
CT2898 t2898 0 0.1f
CT2899 t2899 0 0.1f
M7691 t2897 nw949 vdd vdd pch w=2u l=180n
M7692 t2897 nw948 vdd vdd pch w=2u l=180n
CT2900 t2900 0 0.1f
M7693 t2897 nw949 t2900 0 nch w=1u l=180n
M7694 t2900 nw948 0 0 nch w=1u l=180n
M7695 t2898 nw949 vdd vdd pch w=2u l=180n
M7696 t2898 t2897 vdd vdd pch w=2u l=180n
CT2901 t2901 0 0.1f
M7697 t2898 nw949 t2901 0 nch w=1u l=180n
M7698 t2901 t2897 0 0 nch w=1u l=180n
M7699 t2899 nw948 vdd vdd pch w=2u l=180n
M7700 t2899 t2897 vdd vdd pch w=2u l=180n
CT2902 t2902 0 0.1f
M7701 t2899 nw948 t2902 0 nch w=1u l=180n
M7702 t2902 t2897 0 0 nch w=1u l=180n
M7703 nw950 t2898 vdd vdd pch w=2u l=180n
M7704 nw950 t2899 vdd vdd pch w=2u l=180n
CT2903 t2903 0 0.1f
M7705 nw950 t2898 t2903 0 nch w=1u l=180n
M7706 t2903 t2899 0 0 nch w=1u l=180n
Cnw950 nw950 0 2f
M7707 nw951 nw162 vdd vdd pch w=2u l=180n
M7708 nw951 nw878 vdd vdd pch w=2u l=180n
CT2904 t2904 0 0.1f
M7709 nw951 nw162 t2904 0 nch w=1u l=180n
M7710 t2904 nw878 0 0 nch w=1u l=180n
Cnw951 nw951 0 2f
M7711 nw952 nw949 vdd vdd pch w=2u l=180n
M7712 nw952 nw948 vdd vdd pch w=2u l=180n
CT2905 t2905 0 0.1f
M7713 nw952 nw949 t2905 0 nch w=1u l=180n
M7714 t2905 nw948 0 0 nch w=1u l=180n
Cnw952 nw952 0 2f
M7715 nw953 nw951 vdd vdd pch w=2u l=180n
M7716 nw953 nw952 vdd vdd pch w=2u l=180n
CT2906 t2906 0 0.1f
M7717 nw953 nw951 t2906 0 nch w=1u l=180n
M7718 t2906 nw952 0 0 nch w=1u l=180n
Cnw953 nw953 0 2f
CT2907 t2907 0 0.1f
CT2908 t2908 0 0.1f
CT2909 t2909 0 0.1f
M7719 t2907 nw163 vdd vdd pch w=2u l=180n
M7720 t2907 nw883 vdd vdd pch w=2u l=180n
CT2910 t2910 0 0.1f
M7721 t2907 nw163 t2910 0 nch w=1u l=180n
M7722 t2910 nw883 0 0 nch w=1u l=180n
M7723 t2908 nw163 vdd vdd pch w=2u l=180n
M7724 t2908 t2907 vdd vdd pch w=2u l=180n
CT2911 t2911 0 0.1f
M7725 t2908 nw163 t2911 0 nch w=1u l=180n
M7726 t2911 t2907 0 0 nch w=1u l=180n
M7727 t2909 nw883 vdd vdd pch w=2u l=180n
M7728 t2909 t2907 vdd vdd pch w=2u l=180n
CT2912 t2912 0 0.1f
M7729 t2909 nw883 t2912 0 nch w=1u l=180n
M7730 t2912 t2907 0 0 nch w=1u l=180n
M7731 nw954 t2908 vdd vdd pch w=2u l=180n
M7732 nw954 t2909 vdd vdd pch w=2u l=180n
CT2913 t2913 0 0.1f
M7733 nw954 t2908 t2913 0 nch w=1u l=180n
M7734 t2913 t2909 0 0 nch w=1u l=180n
Cnw954 nw954 0 2f
CT2914 t2914 0 0.1f
CT2915 t2915 0 0.1f
CT2916 t2916 0 0.1f
M7735 t2914 nw954 vdd vdd pch w=2u l=180n
M7736 t2914 nw953 vdd vdd pch w=2u l=180n
CT2917 t2917 0 0.1f
M7737 t2914 nw954 t2917 0 nch w=1u l=180n
M7738 t2917 nw953 0 0 nch w=1u l=180n
M7739 t2915 nw954 vdd vdd pch w=2u l=180n
M7740 t2915 t2914 vdd vdd pch w=2u l=180n
CT2918 t2918 0 0.1f
M7741 t2915 nw954 t2918 0 nch w=1u l=180n
M7742 t2918 t2914 0 0 nch w=1u l=180n
M7743 t2916 nw953 vdd vdd pch w=2u l=180n
M7744 t2916 t2914 vdd vdd pch w=2u l=180n
CT2919 t2919 0 0.1f
M7745 t2916 nw953 t2919 0 nch w=1u l=180n
M7746 t2919 t2914 0 0 nch w=1u l=180n
M7747 nw955 t2915 vdd vdd pch w=2u l=180n
M7748 nw955 t2916 vdd vdd pch w=2u l=180n
CT2920 t2920 0 0.1f
M7749 nw955 t2915 t2920 0 nch w=1u l=180n
M7750 t2920 t2916 0 0 nch w=1u l=180n
Cnw955 nw955 0 2f
M7751 nw956 nw163 vdd vdd pch w=2u l=180n
M7752 nw956 nw883 vdd vdd pch w=2u l=180n
CT2921 t2921 0 0.1f
M7753 nw956 nw163 t2921 0 nch w=1u l=180n
M7754 t2921 nw883 0 0 nch w=1u l=180n
Cnw956 nw956 0 2f
M7755 nw957 nw954 vdd vdd pch w=2u l=180n
M7756 nw957 nw953 vdd vdd pch w=2u l=180n
CT2922 t2922 0 0.1f
M7757 nw957 nw954 t2922 0 nch w=1u l=180n
M7758 t2922 nw953 0 0 nch w=1u l=180n
Cnw957 nw957 0 2f
M7759 nw958 nw956 vdd vdd pch w=2u l=180n
M7760 nw958 nw957 vdd vdd pch w=2u l=180n
CT2923 t2923 0 0.1f
M7761 nw958 nw956 t2923 0 nch w=1u l=180n
M7762 t2923 nw957 0 0 nch w=1u l=180n
Cnw958 nw958 0 2f
CT2924 t2924 0 0.1f
CT2925 t2925 0 0.1f
CT2926 t2926 0 0.1f
M7763 t2924 nw164 vdd vdd pch w=2u l=180n
M7764 t2924 nw888 vdd vdd pch w=2u l=180n
CT2927 t2927 0 0.1f
M7765 t2924 nw164 t2927 0 nch w=1u l=180n
M7766 t2927 nw888 0 0 nch w=1u l=180n
M7767 t2925 nw164 vdd vdd pch w=2u l=180n
M7768 t2925 t2924 vdd vdd pch w=2u l=180n
CT2928 t2928 0 0.1f
M7769 t2925 nw164 t2928 0 nch w=1u l=180n
M7770 t2928 t2924 0 0 nch w=1u l=180n
M7771 t2926 nw888 vdd vdd pch w=2u l=180n
M7772 t2926 t2924 vdd vdd pch w=2u l=180n
CT2929 t2929 0 0.1f
M7773 t2926 nw888 t2929 0 nch w=1u l=180n
M7774 t2929 t2924 0 0 nch w=1u l=180n
M7775 nw959 t2925 vdd vdd pch w=2u l=180n
M7776 nw959 t2926 vdd vdd pch w=2u l=180n
CT2930 t2930 0 0.1f
M7777 nw959 t2925 t2930 0 nch w=1u l=180n
M7778 t2930 t2926 0 0 nch w=1u l=180n
Cnw959 nw959 0 2f
CT2931 t2931 0 0.1f
CT2932 t2932 0 0.1f
CT2933 t2933 0 0.1f
M7779 t2931 nw959 vdd vdd pch w=2u l=180n
M7780 t2931 nw958 vdd vdd pch w=2u l=180n
CT2934 t2934 0 0.1f
M7781 t2931 nw959 t2934 0 nch w=1u l=180n
M7782 t2934 nw958 0 0 nch w=1u l=180n
M7783 t2932 nw959 vdd vdd pch w=2u l=180n
M7784 t2932 t2931 vdd vdd pch w=2u l=180n
CT2935 t2935 0 0.1f
M7785 t2932 nw959 t2935 0 nch w=1u l=180n
M7786 t2935 t2931 0 0 nch w=1u l=180n
M7787 t2933 nw958 vdd vdd pch w=2u l=180n
M7788 t2933 t2931 vdd vdd pch w=2u l=180n
CT2936 t2936 0 0.1f
M7789 t2933 nw958 t2936 0 nch w=1u l=180n
M7790 t2936 t2931 0 0 nch w=1u l=180n
M7791 nw960 t2932 vdd vdd pch w=2u l=180n
M7792 nw960 t2933 vdd vdd pch w=2u l=180n
CT2937 t2937 0 0.1f
M7793 nw960 t2932 t2937 0 nch w=1u l=180n
M7794 t2937 t2933 0 0 nch w=1u l=180n
Cnw960 nw960 0 2f
M7795 nw961 nw164 vdd vdd pch w=2u l=180n
M7796 nw961 nw888 vdd vdd pch w=2u l=180n
CT2938 t2938 0 0.1f
M7797 nw961 nw164 t2938 0 nch w=1u l=180n
M7798 t2938 nw888 0 0 nch w=1u l=180n
Cnw961 nw961 0 2f
M7799 nw962 nw959 vdd vdd pch w=2u l=180n
M7800 nw962 nw958 vdd vdd pch w=2u l=180n
CT2939 t2939 0 0.1f
M7801 nw962 nw959 t2939 0 nch w=1u l=180n
M7802 t2939 nw958 0 0 nch w=1u l=180n
Cnw962 nw962 0 2f
M7803 nw963 nw961 vdd vdd pch w=2u l=180n
M7804 nw963 nw962 vdd vdd pch w=2u l=180n
CT2940 t2940 0 0.1f
M7805 nw963 nw961 t2940 0 nch w=1u l=180n
M7806 t2940 nw962 0 0 nch w=1u l=180n
Cnw963 nw963 0 2f
CT2941 t2941 0 0.1f
CT2942 t2942 0 0.1f
CT2943 t2943 0 0.1f
M7807 t2941 nw165 vdd vdd pch w=2u l=180n
M7808 t2941 nw893 vdd vdd pch w=2u l=180n
CT2944 t2944 0 0.1f
M7809 t2941 nw165 t2944 0 nch w=1u l=180n
M7810 t2944 nw893 0 0 nch w=1u l=180n
M7811 t2942 nw165 vdd vdd pch w=2u l=180n
M7812 t2942 t2941 vdd vdd pch w=2u l=180n
CT2945 t2945 0 0.1f
M7813 t2942 nw165 t2945 0 nch w=1u l=180n
M7814 t2945 t2941 0 0 nch w=1u l=180n
M7815 t2943 nw893 vdd vdd pch w=2u l=180n
M7816 t2943 t2941 vdd vdd pch w=2u l=180n
CT2946 t2946 0 0.1f
M7817 t2943 nw893 t2946 0 nch w=1u l=180n
M7818 t2946 t2941 0 0 nch w=1u l=180n
M7819 nw964 t2942 vdd vdd pch w=2u l=180n
M7820 nw964 t2943 vdd vdd pch w=2u l=180n
CT2947 t2947 0 0.1f
M7821 nw964 t2942 t2947 0 nch w=1u l=180n
M7822 t2947 t2943 0 0 nch w=1u l=180n
Cnw964 nw964 0 2f
CT2948 t2948 0 0.1f
CT2949 t2949 0 0.1f
CT2950 t2950 0 0.1f
M7823 t2948 nw964 vdd vdd pch w=2u l=180n
M7824 t2948 nw963 vdd vdd pch w=2u l=180n
CT2951 t2951 0 0.1f
M7825 t2948 nw964 t2951 0 nch w=1u l=180n
M7826 t2951 nw963 0 0 nch w=1u l=180n
M7827 t2949 nw964 vdd vdd pch w=2u l=180n
M7828 t2949 t2948 vdd vdd pch w=2u l=180n
CT2952 t2952 0 0.1f
M7829 t2949 nw964 t2952 0 nch w=1u l=180n
M7830 t2952 t2948 0 0 nch w=1u l=180n
M7831 t2950 nw963 vdd vdd pch w=2u l=180n
M7832 t2950 t2948 vdd vdd pch w=2u l=180n
CT2953 t2953 0 0.1f
M7833 t2950 nw963 t2953 0 nch w=1u l=180n
M7834 t2953 t2948 0 0 nch w=1u l=180n
M7835 nw965 t2949 vdd vdd pch w=2u l=180n
M7836 nw965 t2950 vdd vdd pch w=2u l=180n
CT2954 t2954 0 0.1f
M7837 nw965 t2949 t2954 0 nch w=1u l=180n
M7838 t2954 t2950 0 0 nch w=1u l=180n
Cnw965 nw965 0 2f
M7839 nw966 nw165 vdd vdd pch w=2u l=180n
M7840 nw966 nw893 vdd vdd pch w=2u l=180n
CT2955 t2955 0 0.1f
M7841 nw966 nw165 t2955 0 nch w=1u l=180n
M7842 t2955 nw893 0 0 nch w=1u l=180n
Cnw966 nw966 0 2f
M7843 nw967 nw964 vdd vdd pch w=2u l=180n
M7844 nw967 nw963 vdd vdd pch w=2u l=180n
CT2956 t2956 0 0.1f
M7845 nw967 nw964 t2956 0 nch w=1u l=180n
M7846 t2956 nw963 0 0 nch w=1u l=180n
Cnw967 nw967 0 2f
M7847 nw968 nw966 vdd vdd pch w=2u l=180n
M7848 nw968 nw967 vdd vdd pch w=2u l=180n
CT2957 t2957 0 0.1f
M7849 nw968 nw966 t2957 0 nch w=1u l=180n
M7850 t2957 nw967 0 0 nch w=1u l=180n
Cnw968 nw968 0 2f
CT2958 t2958 0 0.1f
CT2959 t2959 0 0.1f
CT2960 t2960 0 0.1f
M7851 t2958 nw166 vdd vdd pch w=2u l=180n
M7852 t2958 nw898 vdd vdd pch w=2u l=180n
CT2961 t2961 0 0.1f
M7853 t2958 nw166 t2961 0 nch w=1u l=180n
M7854 t2961 nw898 0 0 nch w=1u l=180n
M7855 t2959 nw166 vdd vdd pch w=2u l=180n
M7856 t2959 t2958 vdd vdd pch w=2u l=180n
CT2962 t2962 0 0.1f
M7857 t2959 nw166 t2962 0 nch w=1u l=180n
M7858 t2962 t2958 0 0 nch w=1u l=180n
M7859 t2960 nw898 vdd vdd pch w=2u l=180n
M7860 t2960 t2958 vdd vdd pch w=2u l=180n
CT2963 t2963 0 0.1f
M7861 t2960 nw898 t2963 0 nch w=1u l=180n
M7862 t2963 t2958 0 0 nch w=1u l=180n
M7863 nw969 t2959 vdd vdd pch w=2u l=180n
M7864 nw969 t2960 vdd vdd pch w=2u l=180n
CT2964 t2964 0 0.1f
M7865 nw969 t2959 t2964 0 nch w=1u l=180n
M7866 t2964 t2960 0 0 nch w=1u l=180n
Cnw969 nw969 0 2f
CT2965 t2965 0 0.1f
CT2966 t2966 0 0.1f
CT2967 t2967 0 0.1f
M7867 t2965 nw969 vdd vdd pch w=2u l=180n
M7868 t2965 nw968 vdd vdd pch w=2u l=180n
CT2968 t2968 0 0.1f
M7869 t2965 nw969 t2968 0 nch w=1u l=180n
M7870 t2968 nw968 0 0 nch w=1u l=180n
M7871 t2966 nw969 vdd vdd pch w=2u l=180n
M7872 t2966 t2965 vdd vdd pch w=2u l=180n
CT2969 t2969 0 0.1f
M7873 t2966 nw969 t2969 0 nch w=1u l=180n
M7874 t2969 t2965 0 0 nch w=1u l=180n
M7875 t2967 nw968 vdd vdd pch w=2u l=180n
M7876 t2967 t2965 vdd vdd pch w=2u l=180n
CT2970 t2970 0 0.1f
M7877 t2967 nw968 t2970 0 nch w=1u l=180n
M7878 t2970 t2965 0 0 nch w=1u l=180n
M7879 nw970 t2966 vdd vdd pch w=2u l=180n
M7880 nw970 t2967 vdd vdd pch w=2u l=180n
CT2971 t2971 0 0.1f
M7881 nw970 t2966 t2971 0 nch w=1u l=180n
M7882 t2971 t2967 0 0 nch w=1u l=180n
Cnw970 nw970 0 2f
M7883 nw971 nw166 vdd vdd pch w=2u l=180n
M7884 nw971 nw898 vdd vdd pch w=2u l=180n
CT2972 t2972 0 0.1f
M7885 nw971 nw166 t2972 0 nch w=1u l=180n
M7886 t2972 nw898 0 0 nch w=1u l=180n
Cnw971 nw971 0 2f
M7887 nw972 nw969 vdd vdd pch w=2u l=180n
M7888 nw972 nw968 vdd vdd pch w=2u l=180n
CT2973 t2973 0 0.1f
M7889 nw972 nw969 t2973 0 nch w=1u l=180n
M7890 t2973 nw968 0 0 nch w=1u l=180n
Cnw972 nw972 0 2f
M7891 nw973 nw971 vdd vdd pch w=2u l=180n
M7892 nw973 nw972 vdd vdd pch w=2u l=180n
CT2974 t2974 0 0.1f
M7893 nw973 nw971 t2974 0 nch w=1u l=180n
M7894 t2974 nw972 0 0 nch w=1u l=180n
Cnw973 nw973 0 2f
CT2975 t2975 0 0.1f
CT2976 t2976 0 0.1f
CT2977 t2977 0 0.1f
M7895 t2975 nw167 vdd vdd pch w=2u l=180n
M7896 t2975 nw903 vdd vdd pch w=2u l=180n
CT2978 t2978 0 0.1f
M7897 t2975 nw167 t2978 0 nch w=1u l=180n
M7898 t2978 nw903 0 0 nch w=1u l=180n
M7899 t2976 nw167 vdd vdd pch w=2u l=180n
M7900 t2976 t2975 vdd vdd pch w=2u l=180n
CT2979 t2979 0 0.1f
M7901 t2976 nw167 t2979 0 nch w=1u l=180n
M7902 t2979 t2975 0 0 nch w=1u l=180n
M7903 t2977 nw903 vdd vdd pch w=2u l=180n
M7904 t2977 t2975 vdd vdd pch w=2u l=180n
CT2980 t2980 0 0.1f
M7905 t2977 nw903 t2980 0 nch w=1u l=180n
M7906 t2980 t2975 0 0 nch w=1u l=180n
M7907 nw974 t2976 vdd vdd pch w=2u l=180n
M7908 nw974 t2977 vdd vdd pch w=2u l=180n
CT2981 t2981 0 0.1f
M7909 nw974 t2976 t2981 0 nch w=1u l=180n
M7910 t2981 t2977 0 0 nch w=1u l=180n
Cnw974 nw974 0 2f
CT2982 t2982 0 0.1f
CT2983 t2983 0 0.1f
CT2984 t2984 0 0.1f
M7911 t2982 nw974 vdd vdd pch w=2u l=180n
M7912 t2982 nw973 vdd vdd pch w=2u l=180n
CT2985 t2985 0 0.1f
M7913 t2982 nw974 t2985 0 nch w=1u l=180n
M7914 t2985 nw973 0 0 nch w=1u l=180n
M7915 t2983 nw974 vdd vdd pch w=2u l=180n
M7916 t2983 t2982 vdd vdd pch w=2u l=180n
CT2986 t2986 0 0.1f
M7917 t2983 nw974 t2986 0 nch w=1u l=180n
M7918 t2986 t2982 0 0 nch w=1u l=180n
M7919 t2984 nw973 vdd vdd pch w=2u l=180n
M7920 t2984 t2982 vdd vdd pch w=2u l=180n
CT2987 t2987 0 0.1f
M7921 t2984 nw973 t2987 0 nch w=1u l=180n
M7922 t2987 t2982 0 0 nch w=1u l=180n
M7923 nw975 t2983 vdd vdd pch w=2u l=180n
M7924 nw975 t2984 vdd vdd pch w=2u l=180n
CT2988 t2988 0 0.1f
M7925 nw975 t2983 t2988 0 nch w=1u l=180n
M7926 t2988 t2984 0 0 nch w=1u l=180n
Cnw975 nw975 0 2f
M7927 nw976 nw167 vdd vdd pch w=2u l=180n
M7928 nw976 nw903 vdd vdd pch w=2u l=180n
CT2989 t2989 0 0.1f
M7929 nw976 nw167 t2989 0 nch w=1u l=180n
M7930 t2989 nw903 0 0 nch w=1u l=180n
Cnw976 nw976 0 2f
M7931 nw977 nw974 vdd vdd pch w=2u l=180n
M7932 nw977 nw973 vdd vdd pch w=2u l=180n
CT2990 t2990 0 0.1f
M7933 nw977 nw974 t2990 0 nch w=1u l=180n
M7934 t2990 nw973 0 0 nch w=1u l=180n
Cnw977 nw977 0 2f
M7935 nw978 nw976 vdd vdd pch w=2u l=180n
M7936 nw978 nw977 vdd vdd pch w=2u l=180n
CT2991 t2991 0 0.1f
M7937 nw978 nw976 t2991 0 nch w=1u l=180n
M7938 t2991 nw977 0 0 nch w=1u l=180n
Cnw978 nw978 0 2f
CT2992 t2992 0 0.1f
CT2993 t2993 0 0.1f
CT2994 t2994 0 0.1f
M7939 t2992 nw168 vdd vdd pch w=2u l=180n
M7940 t2992 nw908 vdd vdd pch w=2u l=180n
CT2995 t2995 0 0.1f
M7941 t2992 nw168 t2995 0 nch w=1u l=180n
M7942 t2995 nw908 0 0 nch w=1u l=180n
M7943 t2993 nw168 vdd vdd pch w=2u l=180n
M7944 t2993 t2992 vdd vdd pch w=2u l=180n
CT2996 t2996 0 0.1f
M7945 t2993 nw168 t2996 0 nch w=1u l=180n
M7946 t2996 t2992 0 0 nch w=1u l=180n
M7947 t2994 nw908 vdd vdd pch w=2u l=180n
M7948 t2994 t2992 vdd vdd pch w=2u l=180n
CT2997 t2997 0 0.1f
M7949 t2994 nw908 t2997 0 nch w=1u l=180n
M7950 t2997 t2992 0 0 nch w=1u l=180n
M7951 nw979 t2993 vdd vdd pch w=2u l=180n
M7952 nw979 t2994 vdd vdd pch w=2u l=180n
CT2998 t2998 0 0.1f
M7953 nw979 t2993 t2998 0 nch w=1u l=180n
M7954 t2998 t2994 0 0 nch w=1u l=180n
Cnw979 nw979 0 2f
CT2999 t2999 0 0.1f
CT3000 t3000 0 0.1f
CT3001 t3001 0 0.1f
M7955 t2999 nw979 vdd vdd pch w=2u l=180n
M7956 t2999 nw978 vdd vdd pch w=2u l=180n
CT3002 t3002 0 0.1f
M7957 t2999 nw979 t3002 0 nch w=1u l=180n
M7958 t3002 nw978 0 0 nch w=1u l=180n
M7959 t3000 nw979 vdd vdd pch w=2u l=180n
M7960 t3000 t2999 vdd vdd pch w=2u l=180n
CT3003 t3003 0 0.1f
M7961 t3000 nw979 t3003 0 nch w=1u l=180n
M7962 t3003 t2999 0 0 nch w=1u l=180n
M7963 t3001 nw978 vdd vdd pch w=2u l=180n
M7964 t3001 t2999 vdd vdd pch w=2u l=180n
CT3004 t3004 0 0.1f
M7965 t3001 nw978 t3004 0 nch w=1u l=180n
M7966 t3004 t2999 0 0 nch w=1u l=180n
M7967 nw980 t3000 vdd vdd pch w=2u l=180n
M7968 nw980 t3001 vdd vdd pch w=2u l=180n
CT3005 t3005 0 0.1f
M7969 nw980 t3000 t3005 0 nch w=1u l=180n
M7970 t3005 t3001 0 0 nch w=1u l=180n
Cnw980 nw980 0 2f
M7971 nw981 nw168 vdd vdd pch w=2u l=180n
M7972 nw981 nw908 vdd vdd pch w=2u l=180n
CT3006 t3006 0 0.1f
M7973 nw981 nw168 t3006 0 nch w=1u l=180n
M7974 t3006 nw908 0 0 nch w=1u l=180n
Cnw981 nw981 0 2f
M7975 nw982 nw979 vdd vdd pch w=2u l=180n
M7976 nw982 nw978 vdd vdd pch w=2u l=180n
CT3007 t3007 0 0.1f
M7977 nw982 nw979 t3007 0 nch w=1u l=180n
M7978 t3007 nw978 0 0 nch w=1u l=180n
Cnw982 nw982 0 2f
M7979 nw983 nw981 vdd vdd pch w=2u l=180n
M7980 nw983 nw982 vdd vdd pch w=2u l=180n
CT3008 t3008 0 0.1f
M7981 nw983 nw981 t3008 0 nch w=1u l=180n
M7982 t3008 nw982 0 0 nch w=1u l=180n
Cnw983 nw983 0 2f
CT3009 t3009 0 0.1f
CT3010 t3010 0 0.1f
CT3011 t3011 0 0.1f
M7983 t3009 nw169 vdd vdd pch w=2u l=180n
M7984 t3009 nw913 vdd vdd pch w=2u l=180n
CT3012 t3012 0 0.1f
M7985 t3009 nw169 t3012 0 nch w=1u l=180n
M7986 t3012 nw913 0 0 nch w=1u l=180n
M7987 t3010 nw169 vdd vdd pch w=2u l=180n
M7988 t3010 t3009 vdd vdd pch w=2u l=180n
CT3013 t3013 0 0.1f
M7989 t3010 nw169 t3013 0 nch w=1u l=180n
M7990 t3013 t3009 0 0 nch w=1u l=180n
M7991 t3011 nw913 vdd vdd pch w=2u l=180n
M7992 t3011 t3009 vdd vdd pch w=2u l=180n
CT3014 t3014 0 0.1f
M7993 t3011 nw913 t3014 0 nch w=1u l=180n
M7994 t3014 t3009 0 0 nch w=1u l=180n
M7995 nw984 t3010 vdd vdd pch w=2u l=180n
M7996 nw984 t3011 vdd vdd pch w=2u l=180n
CT3015 t3015 0 0.1f
M7997 nw984 t3010 t3015 0 nch w=1u l=180n
M7998 t3015 t3011 0 0 nch w=1u l=180n
Cnw984 nw984 0 2f
CT3016 t3016 0 0.1f
CT3017 t3017 0 0.1f
CT3018 t3018 0 0.1f
M7999 t3016 nw984 vdd vdd pch w=2u l=180n
M8000 t3016 nw983 vdd vdd pch w=2u l=180n
CT3019 t3019 0 0.1f
M8001 t3016 nw984 t3019 0 nch w=1u l=180n
M8002 t3019 nw983 0 0 nch w=1u l=180n
M8003 t3017 nw984 vdd vdd pch w=2u l=180n
M8004 t3017 t3016 vdd vdd pch w=2u l=180n
CT3020 t3020 0 0.1f
M8005 t3017 nw984 t3020 0 nch w=1u l=180n
M8006 t3020 t3016 0 0 nch w=1u l=180n
M8007 t3018 nw983 vdd vdd pch w=2u l=180n
M8008 t3018 t3016 vdd vdd pch w=2u l=180n
CT3021 t3021 0 0.1f
M8009 t3018 nw983 t3021 0 nch w=1u l=180n
M8010 t3021 t3016 0 0 nch w=1u l=180n
M8011 nw985 t3017 vdd vdd pch w=2u l=180n
M8012 nw985 t3018 vdd vdd pch w=2u l=180n
CT3022 t3022 0 0.1f
M8013 nw985 t3017 t3022 0 nch w=1u l=180n
M8014 t3022 t3018 0 0 nch w=1u l=180n
Cnw985 nw985 0 2f
M8015 nw986 nw169 vdd vdd pch w=2u l=180n
M8016 nw986 nw913 vdd vdd pch w=2u l=180n
CT3023 t3023 0 0.1f
M8017 nw986 nw169 t3023 0 nch w=1u l=180n
M8018 t3023 nw913 0 0 nch w=1u l=180n
Cnw986 nw986 0 2f
M8019 nw987 nw984 vdd vdd pch w=2u l=180n
M8020 nw987 nw983 vdd vdd pch w=2u l=180n
CT3024 t3024 0 0.1f
M8021 nw987 nw984 t3024 0 nch w=1u l=180n
M8022 t3024 nw983 0 0 nch w=1u l=180n
Cnw987 nw987 0 2f
M8023 nw988 nw986 vdd vdd pch w=2u l=180n
M8024 nw988 nw987 vdd vdd pch w=2u l=180n
CT3025 t3025 0 0.1f
M8025 nw988 nw986 t3025 0 nch w=1u l=180n
M8026 t3025 nw987 0 0 nch w=1u l=180n
Cnw988 nw988 0 2f
CT3026 t3026 0 0.1f
CT3027 t3027 0 0.1f
CT3028 t3028 0 0.1f
M8027 t3026 nw170 vdd vdd pch w=2u l=180n
M8028 t3026 nw918 vdd vdd pch w=2u l=180n
CT3029 t3029 0 0.1f
M8029 t3026 nw170 t3029 0 nch w=1u l=180n
M8030 t3029 nw918 0 0 nch w=1u l=180n
M8031 t3027 nw170 vdd vdd pch w=2u l=180n
M8032 t3027 t3026 vdd vdd pch w=2u l=180n
CT3030 t3030 0 0.1f
M8033 t3027 nw170 t3030 0 nch w=1u l=180n
M8034 t3030 t3026 0 0 nch w=1u l=180n
M8035 t3028 nw918 vdd vdd pch w=2u l=180n
M8036 t3028 t3026 vdd vdd pch w=2u l=180n
CT3031 t3031 0 0.1f
M8037 t3028 nw918 t3031 0 nch w=1u l=180n
M8038 t3031 t3026 0 0 nch w=1u l=180n
M8039 nw989 t3027 vdd vdd pch w=2u l=180n
M8040 nw989 t3028 vdd vdd pch w=2u l=180n
CT3032 t3032 0 0.1f
M8041 nw989 t3027 t3032 0 nch w=1u l=180n
M8042 t3032 t3028 0 0 nch w=1u l=180n
Cnw989 nw989 0 2f
CT3033 t3033 0 0.1f
CT3034 t3034 0 0.1f
CT3035 t3035 0 0.1f
M8043 t3033 nw989 vdd vdd pch w=2u l=180n
M8044 t3033 nw988 vdd vdd pch w=2u l=180n
CT3036 t3036 0 0.1f
M8045 t3033 nw989 t3036 0 nch w=1u l=180n
M8046 t3036 nw988 0 0 nch w=1u l=180n
M8047 t3034 nw989 vdd vdd pch w=2u l=180n
M8048 t3034 t3033 vdd vdd pch w=2u l=180n
CT3037 t3037 0 0.1f
M8049 t3034 nw989 t3037 0 nch w=1u l=180n
M8050 t3037 t3033 0 0 nch w=1u l=180n
M8051 t3035 nw988 vdd vdd pch w=2u l=180n
M8052 t3035 t3033 vdd vdd pch w=2u l=180n
CT3038 t3038 0 0.1f
M8053 t3035 nw988 t3038 0 nch w=1u l=180n
M8054 t3038 t3033 0 0 nch w=1u l=180n
M8055 nw990 t3034 vdd vdd pch w=2u l=180n
M8056 nw990 t3035 vdd vdd pch w=2u l=180n
CT3039 t3039 0 0.1f
M8057 nw990 t3034 t3039 0 nch w=1u l=180n
M8058 t3039 t3035 0 0 nch w=1u l=180n
Cnw990 nw990 0 2f
M8059 nw991 nw170 vdd vdd pch w=2u l=180n
M8060 nw991 nw918 vdd vdd pch w=2u l=180n
CT3040 t3040 0 0.1f
M8061 nw991 nw170 t3040 0 nch w=1u l=180n
M8062 t3040 nw918 0 0 nch w=1u l=180n
Cnw991 nw991 0 2f
M8063 nw992 nw989 vdd vdd pch w=2u l=180n
M8064 nw992 nw988 vdd vdd pch w=2u l=180n
CT3041 t3041 0 0.1f
M8065 nw992 nw989 t3041 0 nch w=1u l=180n
M8066 t3041 nw988 0 0 nch w=1u l=180n
Cnw992 nw992 0 2f
M8067 nw993 nw991 vdd vdd pch w=2u l=180n
M8068 nw993 nw992 vdd vdd pch w=2u l=180n
CT3042 t3042 0 0.1f
M8069 nw993 nw991 t3042 0 nch w=1u l=180n
M8070 t3042 nw992 0 0 nch w=1u l=180n
Cnw993 nw993 0 2f
CT3043 t3043 0 0.1f
CT3044 t3044 0 0.1f
CT3045 t3045 0 0.1f
M8071 t3043 nw171 vdd vdd pch w=2u l=180n
M8072 t3043 nw923 vdd vdd pch w=2u l=180n
CT3046 t3046 0 0.1f
M8073 t3043 nw171 t3046 0 nch w=1u l=180n
M8074 t3046 nw923 0 0 nch w=1u l=180n
M8075 t3044 nw171 vdd vdd pch w=2u l=180n
M8076 t3044 t3043 vdd vdd pch w=2u l=180n
CT3047 t3047 0 0.1f
M8077 t3044 nw171 t3047 0 nch w=1u l=180n
M8078 t3047 t3043 0 0 nch w=1u l=180n
M8079 t3045 nw923 vdd vdd pch w=2u l=180n
M8080 t3045 t3043 vdd vdd pch w=2u l=180n
CT3048 t3048 0 0.1f
M8081 t3045 nw923 t3048 0 nch w=1u l=180n
M8082 t3048 t3043 0 0 nch w=1u l=180n
M8083 nw994 t3044 vdd vdd pch w=2u l=180n
M8084 nw994 t3045 vdd vdd pch w=2u l=180n
CT3049 t3049 0 0.1f
M8085 nw994 t3044 t3049 0 nch w=1u l=180n
M8086 t3049 t3045 0 0 nch w=1u l=180n
Cnw994 nw994 0 2f
CT3050 t3050 0 0.1f
CT3051 t3051 0 0.1f
CT3052 t3052 0 0.1f
M8087 t3050 nw994 vdd vdd pch w=2u l=180n
M8088 t3050 nw993 vdd vdd pch w=2u l=180n
CT3053 t3053 0 0.1f
M8089 t3050 nw994 t3053 0 nch w=1u l=180n
M8090 t3053 nw993 0 0 nch w=1u l=180n
M8091 t3051 nw994 vdd vdd pch w=2u l=180n
M8092 t3051 t3050 vdd vdd pch w=2u l=180n
CT3054 t3054 0 0.1f
M8093 t3051 nw994 t3054 0 nch w=1u l=180n
M8094 t3054 t3050 0 0 nch w=1u l=180n
M8095 t3052 nw993 vdd vdd pch w=2u l=180n
M8096 t3052 t3050 vdd vdd pch w=2u l=180n
CT3055 t3055 0 0.1f
M8097 t3052 nw993 t3055 0 nch w=1u l=180n
M8098 t3055 t3050 0 0 nch w=1u l=180n
M8099 nw995 t3051 vdd vdd pch w=2u l=180n
M8100 nw995 t3052 vdd vdd pch w=2u l=180n
CT3056 t3056 0 0.1f
M8101 nw995 t3051 t3056 0 nch w=1u l=180n
M8102 t3056 t3052 0 0 nch w=1u l=180n
Cnw995 nw995 0 2f
M8103 nw996 nw171 vdd vdd pch w=2u l=180n
M8104 nw996 nw923 vdd vdd pch w=2u l=180n
CT3057 t3057 0 0.1f
M8105 nw996 nw171 t3057 0 nch w=1u l=180n
M8106 t3057 nw923 0 0 nch w=1u l=180n
Cnw996 nw996 0 2f
M8107 nw997 nw994 vdd vdd pch w=2u l=180n
M8108 nw997 nw993 vdd vdd pch w=2u l=180n
CT3058 t3058 0 0.1f
M8109 nw997 nw994 t3058 0 nch w=1u l=180n
M8110 t3058 nw993 0 0 nch w=1u l=180n
Cnw997 nw997 0 2f
M8111 nw998 nw996 vdd vdd pch w=2u l=180n
M8112 nw998 nw997 vdd vdd pch w=2u l=180n
CT3059 t3059 0 0.1f
M8113 nw998 nw996 t3059 0 nch w=1u l=180n
M8114 t3059 nw997 0 0 nch w=1u l=180n
Cnw998 nw998 0 2f
CT3060 t3060 0 0.1f
CT3061 t3061 0 0.1f
CT3062 t3062 0 0.1f
M8115 t3060 nw172 vdd vdd pch w=2u l=180n
M8116 t3060 nw928 vdd vdd pch w=2u l=180n
CT3063 t3063 0 0.1f
M8117 t3060 nw172 t3063 0 nch w=1u l=180n
M8118 t3063 nw928 0 0 nch w=1u l=180n
M8119 t3061 nw172 vdd vdd pch w=2u l=180n
M8120 t3061 t3060 vdd vdd pch w=2u l=180n
CT3064 t3064 0 0.1f
M8121 t3061 nw172 t3064 0 nch w=1u l=180n
M8122 t3064 t3060 0 0 nch w=1u l=180n
M8123 t3062 nw928 vdd vdd pch w=2u l=180n
M8124 t3062 t3060 vdd vdd pch w=2u l=180n
CT3065 t3065 0 0.1f
M8125 t3062 nw928 t3065 0 nch w=1u l=180n
M8126 t3065 t3060 0 0 nch w=1u l=180n
M8127 nw999 t3061 vdd vdd pch w=2u l=180n
M8128 nw999 t3062 vdd vdd pch w=2u l=180n
CT3066 t3066 0 0.1f
M8129 nw999 t3061 t3066 0 nch w=1u l=180n
M8130 t3066 t3062 0 0 nch w=1u l=180n
Cnw999 nw999 0 2f
CT3067 t3067 0 0.1f
CT3068 t3068 0 0.1f
CT3069 t3069 0 0.1f
M8131 t3067 nw999 vdd vdd pch w=2u l=180n
M8132 t3067 nw998 vdd vdd pch w=2u l=180n
CT3070 t3070 0 0.1f
M8133 t3067 nw999 t3070 0 nch w=1u l=180n
M8134 t3070 nw998 0 0 nch w=1u l=180n
M8135 t3068 nw999 vdd vdd pch w=2u l=180n
M8136 t3068 t3067 vdd vdd pch w=2u l=180n
CT3071 t3071 0 0.1f
M8137 t3068 nw999 t3071 0 nch w=1u l=180n
M8138 t3071 t3067 0 0 nch w=1u l=180n
M8139 t3069 nw998 vdd vdd pch w=2u l=180n
M8140 t3069 t3067 vdd vdd pch w=2u l=180n
CT3072 t3072 0 0.1f
M8141 t3069 nw998 t3072 0 nch w=1u l=180n
M8142 t3072 t3067 0 0 nch w=1u l=180n
M8143 nw1000 t3068 vdd vdd pch w=2u l=180n
M8144 nw1000 t3069 vdd vdd pch w=2u l=180n
CT3073 t3073 0 0.1f
M8145 nw1000 t3068 t3073 0 nch w=1u l=180n
M8146 t3073 t3069 0 0 nch w=1u l=180n
Cnw1000 nw1000 0 2f
M8147 nw1001 nw172 vdd vdd pch w=2u l=180n
M8148 nw1001 nw928 vdd vdd pch w=2u l=180n
CT3074 t3074 0 0.1f
M8149 nw1001 nw172 t3074 0 nch w=1u l=180n
M8150 t3074 nw928 0 0 nch w=1u l=180n
Cnw1001 nw1001 0 2f
M8151 nw1002 nw999 vdd vdd pch w=2u l=180n
M8152 nw1002 nw998 vdd vdd pch w=2u l=180n
CT3075 t3075 0 0.1f
M8153 nw1002 nw999 t3075 0 nch w=1u l=180n
M8154 t3075 nw998 0 0 nch w=1u l=180n
Cnw1002 nw1002 0 2f
M8155 nw1003 nw1001 vdd vdd pch w=2u l=180n
M8156 nw1003 nw1002 vdd vdd pch w=2u l=180n
CT3076 t3076 0 0.1f
M8157 nw1003 nw1001 t3076 0 nch w=1u l=180n
M8158 t3076 nw1002 0 0 nch w=1u l=180n
Cnw1003 nw1003 0 2f
CT3077 t3077 0 0.1f
CT3078 t3078 0 0.1f
CT3079 t3079 0 0.1f
M8159 t3077 nw173 vdd vdd pch w=2u l=180n
M8160 t3077 nw933 vdd vdd pch w=2u l=180n
CT3080 t3080 0 0.1f
M8161 t3077 nw173 t3080 0 nch w=1u l=180n
M8162 t3080 nw933 0 0 nch w=1u l=180n
M8163 t3078 nw173 vdd vdd pch w=2u l=180n
M8164 t3078 t3077 vdd vdd pch w=2u l=180n
CT3081 t3081 0 0.1f
M8165 t3078 nw173 t3081 0 nch w=1u l=180n
M8166 t3081 t3077 0 0 nch w=1u l=180n
M8167 t3079 nw933 vdd vdd pch w=2u l=180n
M8168 t3079 t3077 vdd vdd pch w=2u l=180n
CT3082 t3082 0 0.1f
M8169 t3079 nw933 t3082 0 nch w=1u l=180n
M8170 t3082 t3077 0 0 nch w=1u l=180n
M8171 nw1004 t3078 vdd vdd pch w=2u l=180n
M8172 nw1004 t3079 vdd vdd pch w=2u l=180n
CT3083 t3083 0 0.1f
M8173 nw1004 t3078 t3083 0 nch w=1u l=180n
M8174 t3083 t3079 0 0 nch w=1u l=180n
Cnw1004 nw1004 0 2f
CT3084 t3084 0 0.1f
CT3085 t3085 0 0.1f
CT3086 t3086 0 0.1f
M8175 t3084 nw1004 vdd vdd pch w=2u l=180n
M8176 t3084 nw1003 vdd vdd pch w=2u l=180n
CT3087 t3087 0 0.1f
M8177 t3084 nw1004 t3087 0 nch w=1u l=180n
M8178 t3087 nw1003 0 0 nch w=1u l=180n
M8179 t3085 nw1004 vdd vdd pch w=2u l=180n
M8180 t3085 t3084 vdd vdd pch w=2u l=180n
CT3088 t3088 0 0.1f
M8181 t3085 nw1004 t3088 0 nch w=1u l=180n
M8182 t3088 t3084 0 0 nch w=1u l=180n
M8183 t3086 nw1003 vdd vdd pch w=2u l=180n
M8184 t3086 t3084 vdd vdd pch w=2u l=180n
CT3089 t3089 0 0.1f
M8185 t3086 nw1003 t3089 0 nch w=1u l=180n
M8186 t3089 t3084 0 0 nch w=1u l=180n
M8187 nw1005 t3085 vdd vdd pch w=2u l=180n
M8188 nw1005 t3086 vdd vdd pch w=2u l=180n
CT3090 t3090 0 0.1f
M8189 nw1005 t3085 t3090 0 nch w=1u l=180n
M8190 t3090 t3086 0 0 nch w=1u l=180n
Cnw1005 nw1005 0 2f
M8191 nw1006 nw173 vdd vdd pch w=2u l=180n
M8192 nw1006 nw933 vdd vdd pch w=2u l=180n
CT3091 t3091 0 0.1f
M8193 nw1006 nw173 t3091 0 nch w=1u l=180n
M8194 t3091 nw933 0 0 nch w=1u l=180n
Cnw1006 nw1006 0 2f
M8195 nw1007 nw1004 vdd vdd pch w=2u l=180n
M8196 nw1007 nw1003 vdd vdd pch w=2u l=180n
CT3092 t3092 0 0.1f
M8197 nw1007 nw1004 t3092 0 nch w=1u l=180n
M8198 t3092 nw1003 0 0 nch w=1u l=180n
Cnw1007 nw1007 0 2f
M8199 nw1008 nw1006 vdd vdd pch w=2u l=180n
M8200 nw1008 nw1007 vdd vdd pch w=2u l=180n
CT3093 t3093 0 0.1f
M8201 nw1008 nw1006 t3093 0 nch w=1u l=180n
M8202 t3093 nw1007 0 0 nch w=1u l=180n
Cnw1008 nw1008 0 2f
CT3094 t3094 0 0.1f
CT3095 t3095 0 0.1f
CT3096 t3096 0 0.1f
M8203 t3094 nw174 vdd vdd pch w=2u l=180n
M8204 t3094 nw938 vdd vdd pch w=2u l=180n
CT3097 t3097 0 0.1f
M8205 t3094 nw174 t3097 0 nch w=1u l=180n
M8206 t3097 nw938 0 0 nch w=1u l=180n
M8207 t3095 nw174 vdd vdd pch w=2u l=180n
M8208 t3095 t3094 vdd vdd pch w=2u l=180n
CT3098 t3098 0 0.1f
M8209 t3095 nw174 t3098 0 nch w=1u l=180n
M8210 t3098 t3094 0 0 nch w=1u l=180n
M8211 t3096 nw938 vdd vdd pch w=2u l=180n
M8212 t3096 t3094 vdd vdd pch w=2u l=180n
CT3099 t3099 0 0.1f
M8213 t3096 nw938 t3099 0 nch w=1u l=180n
M8214 t3099 t3094 0 0 nch w=1u l=180n
M8215 nw1009 t3095 vdd vdd pch w=2u l=180n
M8216 nw1009 t3096 vdd vdd pch w=2u l=180n
CT3100 t3100 0 0.1f
M8217 nw1009 t3095 t3100 0 nch w=1u l=180n
M8218 t3100 t3096 0 0 nch w=1u l=180n
Cnw1009 nw1009 0 2f
CT3101 t3101 0 0.1f
CT3102 t3102 0 0.1f
CT3103 t3103 0 0.1f
M8219 t3101 nw1009 vdd vdd pch w=2u l=180n
M8220 t3101 nw1008 vdd vdd pch w=2u l=180n
CT3104 t3104 0 0.1f
M8221 t3101 nw1009 t3104 0 nch w=1u l=180n
M8222 t3104 nw1008 0 0 nch w=1u l=180n
M8223 t3102 nw1009 vdd vdd pch w=2u l=180n
M8224 t3102 t3101 vdd vdd pch w=2u l=180n
CT3105 t3105 0 0.1f
M8225 t3102 nw1009 t3105 0 nch w=1u l=180n
M8226 t3105 t3101 0 0 nch w=1u l=180n
M8227 t3103 nw1008 vdd vdd pch w=2u l=180n
M8228 t3103 t3101 vdd vdd pch w=2u l=180n
CT3106 t3106 0 0.1f
M8229 t3103 nw1008 t3106 0 nch w=1u l=180n
M8230 t3106 t3101 0 0 nch w=1u l=180n
M8231 nw1010 t3102 vdd vdd pch w=2u l=180n
M8232 nw1010 t3103 vdd vdd pch w=2u l=180n
CT3107 t3107 0 0.1f
M8233 nw1010 t3102 t3107 0 nch w=1u l=180n
M8234 t3107 t3103 0 0 nch w=1u l=180n
Cnw1010 nw1010 0 2f
M8235 nw1011 nw174 vdd vdd pch w=2u l=180n
M8236 nw1011 nw938 vdd vdd pch w=2u l=180n
CT3108 t3108 0 0.1f
M8237 nw1011 nw174 t3108 0 nch w=1u l=180n
M8238 t3108 nw938 0 0 nch w=1u l=180n
Cnw1011 nw1011 0 2f
M8239 nw1012 nw1009 vdd vdd pch w=2u l=180n
M8240 nw1012 nw1008 vdd vdd pch w=2u l=180n
CT3109 t3109 0 0.1f
M8241 nw1012 nw1009 t3109 0 nch w=1u l=180n
M8242 t3109 nw1008 0 0 nch w=1u l=180n
Cnw1012 nw1012 0 2f
M8243 nw1013 nw1011 vdd vdd pch w=2u l=180n
M8244 nw1013 nw1012 vdd vdd pch w=2u l=180n
CT3110 t3110 0 0.1f
M8245 nw1013 nw1011 t3110 0 nch w=1u l=180n
M8246 t3110 nw1012 0 0 nch w=1u l=180n
Cnw1013 nw1013 0 2f
CT3111 t3111 0 0.1f
CT3112 t3112 0 0.1f
CT3113 t3113 0 0.1f
M8247 t3111 nw175 vdd vdd pch w=2u l=180n
M8248 t3111 nw943 vdd vdd pch w=2u l=180n
CT3114 t3114 0 0.1f
M8249 t3111 nw175 t3114 0 nch w=1u l=180n
M8250 t3114 nw943 0 0 nch w=1u l=180n
M8251 t3112 nw175 vdd vdd pch w=2u l=180n
M8252 t3112 t3111 vdd vdd pch w=2u l=180n
CT3115 t3115 0 0.1f
M8253 t3112 nw175 t3115 0 nch w=1u l=180n
M8254 t3115 t3111 0 0 nch w=1u l=180n
M8255 t3113 nw943 vdd vdd pch w=2u l=180n
M8256 t3113 t3111 vdd vdd pch w=2u l=180n
CT3116 t3116 0 0.1f
M8257 t3113 nw943 t3116 0 nch w=1u l=180n
M8258 t3116 t3111 0 0 nch w=1u l=180n
M8259 nw1014 t3112 vdd vdd pch w=2u l=180n
M8260 nw1014 t3113 vdd vdd pch w=2u l=180n
CT3117 t3117 0 0.1f
M8261 nw1014 t3112 t3117 0 nch w=1u l=180n
M8262 t3117 t3113 0 0 nch w=1u l=180n
Cnw1014 nw1014 0 2f
CT3118 t3118 0 0.1f
CT3119 t3119 0 0.1f
CT3120 t3120 0 0.1f
M8263 t3118 nw1014 vdd vdd pch w=2u l=180n
M8264 t3118 nw1013 vdd vdd pch w=2u l=180n
CT3121 t3121 0 0.1f
M8265 t3118 nw1014 t3121 0 nch w=1u l=180n
M8266 t3121 nw1013 0 0 nch w=1u l=180n
M8267 t3119 nw1014 vdd vdd pch w=2u l=180n
M8268 t3119 t3118 vdd vdd pch w=2u l=180n
CT3122 t3122 0 0.1f
M8269 t3119 nw1014 t3122 0 nch w=1u l=180n
M8270 t3122 t3118 0 0 nch w=1u l=180n
M8271 t3120 nw1013 vdd vdd pch w=2u l=180n
M8272 t3120 t3118 vdd vdd pch w=2u l=180n
CT3123 t3123 0 0.1f
M8273 t3120 nw1013 t3123 0 nch w=1u l=180n
M8274 t3123 t3118 0 0 nch w=1u l=180n
M8275 nw1015 t3119 vdd vdd pch w=2u l=180n
M8276 nw1015 t3120 vdd vdd pch w=2u l=180n
CT3124 t3124 0 0.1f
M8277 nw1015 t3119 t3124 0 nch w=1u l=180n
M8278 t3124 t3120 0 0 nch w=1u l=180n
Cnw1015 nw1015 0 2f
M8279 nw1016 nw175 vdd vdd pch w=2u l=180n
M8280 nw1016 nw943 vdd vdd pch w=2u l=180n
CT3125 t3125 0 0.1f
M8281 nw1016 nw175 t3125 0 nch w=1u l=180n
M8282 t3125 nw943 0 0 nch w=1u l=180n
Cnw1016 nw1016 0 2f
M8283 nw1017 nw1014 vdd vdd pch w=2u l=180n
M8284 nw1017 nw1013 vdd vdd pch w=2u l=180n
CT3126 t3126 0 0.1f
M8285 nw1017 nw1014 t3126 0 nch w=1u l=180n
M8286 t3126 nw1013 0 0 nch w=1u l=180n
Cnw1017 nw1017 0 2f
M8287 nw1018 nw1016 vdd vdd pch w=2u l=180n
M8288 nw1018 nw1017 vdd vdd pch w=2u l=180n
CT3127 t3127 0 0.1f
M8289 nw1018 nw1016 t3127 0 nch w=1u l=180n
M8290 t3127 nw1017 0 0 nch w=1u l=180n
Cnw1018 nw1018 0 2f
CT3128 t3128 0 0.1f
CT3129 t3129 0 0.1f
CT3130 t3130 0 0.1f
M8291 t3128 nw176 vdd vdd pch w=2u l=180n
M8292 t3128 nw946 vdd vdd pch w=2u l=180n
CT3131 t3131 0 0.1f
M8293 t3128 nw176 t3131 0 nch w=1u l=180n
M8294 t3131 nw946 0 0 nch w=1u l=180n
M8295 t3129 nw176 vdd vdd pch w=2u l=180n
M8296 t3129 t3128 vdd vdd pch w=2u l=180n
CT3132 t3132 0 0.1f
M8297 t3129 nw176 t3132 0 nch w=1u l=180n
M8298 t3132 t3128 0 0 nch w=1u l=180n
M8299 t3130 nw946 vdd vdd pch w=2u l=180n
M8300 t3130 t3128 vdd vdd pch w=2u l=180n
CT3133 t3133 0 0.1f
M8301 t3130 nw946 t3133 0 nch w=1u l=180n
M8302 t3133 t3128 0 0 nch w=1u l=180n
M8303 nw1019 t3129 vdd vdd pch w=2u l=180n
M8304 nw1019 t3130 vdd vdd pch w=2u l=180n
CT3134 t3134 0 0.1f
M8305 nw1019 t3129 t3134 0 nch w=1u l=180n
M8306 t3134 t3130 0 0 nch w=1u l=180n
Cnw1019 nw1019 0 2f
CT3135 t3135 0 0.1f
CT3136 t3136 0 0.1f
CT3137 t3137 0 0.1f
M8307 t3135 nw1019 vdd vdd pch w=2u l=180n
M8308 t3135 nw1018 vdd vdd pch w=2u l=180n
CT3138 t3138 0 0.1f
M8309 t3135 nw1019 t3138 0 nch w=1u l=180n
M8310 t3138 nw1018 0 0 nch w=1u l=180n
M8311 t3136 nw1019 vdd vdd pch w=2u l=180n
M8312 t3136 t3135 vdd vdd pch w=2u l=180n
CT3139 t3139 0 0.1f
M8313 t3136 nw1019 t3139 0 nch w=1u l=180n
M8314 t3139 t3135 0 0 nch w=1u l=180n
M8315 t3137 nw1018 vdd vdd pch w=2u l=180n
M8316 t3137 t3135 vdd vdd pch w=2u l=180n
CT3140 t3140 0 0.1f
M8317 t3137 nw1018 t3140 0 nch w=1u l=180n
M8318 t3140 t3135 0 0 nch w=1u l=180n
M8319 nw1020 t3136 vdd vdd pch w=2u l=180n
M8320 nw1020 t3137 vdd vdd pch w=2u l=180n
CT3141 t3141 0 0.1f
M8321 nw1020 t3136 t3141 0 nch w=1u l=180n
M8322 t3141 t3137 0 0 nch w=1u l=180n
Cnw1020 nw1020 0 2f
M8323 nw1021 nw176 vdd vdd pch w=2u l=180n
M8324 nw1021 nw946 vdd vdd pch w=2u l=180n
CT3142 t3142 0 0.1f
M8325 nw1021 nw176 t3142 0 nch w=1u l=180n
M8326 t3142 nw946 0 0 nch w=1u l=180n
Cnw1021 nw1021 0 2f
M8327 nw1022 nw1019 vdd vdd pch w=2u l=180n
M8328 nw1022 nw1018 vdd vdd pch w=2u l=180n
CT3143 t3143 0 0.1f
M8329 nw1022 nw1019 t3143 0 nch w=1u l=180n
M8330 t3143 nw1018 0 0 nch w=1u l=180n
Cnw1022 nw1022 0 2f
M8331 nw1023 nw1021 vdd vdd pch w=2u l=180n
M8332 nw1023 nw1022 vdd vdd pch w=2u l=180n
CT3144 t3144 0 0.1f
M8333 nw1023 nw1021 t3144 0 nch w=1u l=180n
M8334 t3144 nw1022 0 0 nch w=1u l=180n
Cnw1023 nw1023 0 2f
CT3145 t3145 0 0.1f
CT3146 t3146 0 0.1f
CT3147 t3147 0 0.1f
M8335 t3145 nw177 vdd vdd pch w=2u l=180n
M8336 t3145 nw950 vdd vdd pch w=2u l=180n
CT3148 t3148 0 0.1f
M8337 t3145 nw177 t3148 0 nch w=1u l=180n
M8338 t3148 nw950 0 0 nch w=1u l=180n
M8339 t3146 nw177 vdd vdd pch w=2u l=180n
M8340 t3146 t3145 vdd vdd pch w=2u l=180n
CT3149 t3149 0 0.1f
M8341 t3146 nw177 t3149 0 nch w=1u l=180n
M8342 t3149 t3145 0 0 nch w=1u l=180n
M8343 t3147 nw950 vdd vdd pch w=2u l=180n
M8344 t3147 t3145 vdd vdd pch w=2u l=180n
CT3150 t3150 0 0.1f
M8345 t3147 nw950 t3150 0 nch w=1u l=180n
M8346 t3150 t3145 0 0 nch w=1u l=180n
M8347 nw1024 t3146 vdd vdd pch w=2u l=180n
M8348 nw1024 t3147 vdd vdd pch w=2u l=180n
CT3151 t3151 0 0.1f
M8349 nw1024 t3146 t3151 0 nch w=1u l=180n
M8350 t3151 t3147 0 0 nch w=1u l=180n
Cnw1024 nw1024 0 2f
CT3152 t3152 0 0.1f
M8351 t3152 nw177 vdd vdd pch w=2u l=180n
M8352 t3152 nw950 vdd vdd pch w=2u l=180n
CT3153 t3153 0 0.1f
M8353 t3152 nw177 t3153 0 nch w=1u l=180n
M8354 t3153 nw950 0 0 nch w=1u l=180n
M8355 nw1025 t3152 vdd vdd pch w=2u l=180n
M8356 nw1025 t3152 0 0 nch w=1u l=180n
Cnw1025 nw1025 0 2f
CT3154 t3154 0 0.1f
CT3155 t3155 0 0.1f
CT3156 t3156 0 0.1f
M8357 t3154 nw178 vdd vdd pch w=2u l=180n
M8358 t3154 nw955 vdd vdd pch w=2u l=180n
CT3157 t3157 0 0.1f
M8359 t3154 nw178 t3157 0 nch w=1u l=180n
M8360 t3157 nw955 0 0 nch w=1u l=180n
M8361 t3155 nw178 vdd vdd pch w=2u l=180n
M8362 t3155 t3154 vdd vdd pch w=2u l=180n
CT3158 t3158 0 0.1f
M8363 t3155 nw178 t3158 0 nch w=1u l=180n
M8364 t3158 t3154 0 0 nch w=1u l=180n
M8365 t3156 nw955 vdd vdd pch w=2u l=180n
M8366 t3156 t3154 vdd vdd pch w=2u l=180n
CT3159 t3159 0 0.1f
M8367 t3156 nw955 t3159 0 nch w=1u l=180n
M8368 t3159 t3154 0 0 nch w=1u l=180n
M8369 nw1026 t3155 vdd vdd pch w=2u l=180n
M8370 nw1026 t3156 vdd vdd pch w=2u l=180n
CT3160 t3160 0 0.1f
M8371 nw1026 t3155 t3160 0 nch w=1u l=180n
M8372 t3160 t3156 0 0 nch w=1u l=180n
Cnw1026 nw1026 0 2f
CT3161 t3161 0 0.1f
CT3162 t3162 0 0.1f
CT3163 t3163 0 0.1f
M8373 t3161 nw1026 vdd vdd pch w=2u l=180n
M8374 t3161 nw1025 vdd vdd pch w=2u l=180n
CT3164 t3164 0 0.1f
M8375 t3161 nw1026 t3164 0 nch w=1u l=180n
M8376 t3164 nw1025 0 0 nch w=1u l=180n
M8377 t3162 nw1026 vdd vdd pch w=2u l=180n
M8378 t3162 t3161 vdd vdd pch w=2u l=180n
CT3165 t3165 0 0.1f
M8379 t3162 nw1026 t3165 0 nch w=1u l=180n
M8380 t3165 t3161 0 0 nch w=1u l=180n
M8381 t3163 nw1025 vdd vdd pch w=2u l=180n
M8382 t3163 t3161 vdd vdd pch w=2u l=180n
CT3166 t3166 0 0.1f
M8383 t3163 nw1025 t3166 0 nch w=1u l=180n
M8384 t3166 t3161 0 0 nch w=1u l=180n
M8385 nw1027 t3162 vdd vdd pch w=2u l=180n
M8386 nw1027 t3163 vdd vdd pch w=2u l=180n
CT3167 t3167 0 0.1f
M8387 nw1027 t3162 t3167 0 nch w=1u l=180n
M8388 t3167 t3163 0 0 nch w=1u l=180n
Cnw1027 nw1027 0 2f
M8389 nw1028 nw178 vdd vdd pch w=2u l=180n
M8390 nw1028 nw955 vdd vdd pch w=2u l=180n
CT3168 t3168 0 0.1f
M8391 nw1028 nw178 t3168 0 nch w=1u l=180n
M8392 t3168 nw955 0 0 nch w=1u l=180n
Cnw1028 nw1028 0 2f
M8393 nw1029 nw1026 vdd vdd pch w=2u l=180n
M8394 nw1029 nw1025 vdd vdd pch w=2u l=180n
CT3169 t3169 0 0.1f
M8395 nw1029 nw1026 t3169 0 nch w=1u l=180n
M8396 t3169 nw1025 0 0 nch w=1u l=180n
Cnw1029 nw1029 0 2f
M8397 nw1030 nw1028 vdd vdd pch w=2u l=180n
M8398 nw1030 nw1029 vdd vdd pch w=2u l=180n
CT3170 t3170 0 0.1f
M8399 nw1030 nw1028 t3170 0 nch w=1u l=180n
M8400 t3170 nw1029 0 0 nch w=1u l=180n
Cnw1030 nw1030 0 2f
CT3171 t3171 0 0.1f
CT3172 t3172 0 0.1f
CT3173 t3173 0 0.1f
M8401 t3171 nw179 vdd vdd pch w=2u l=180n
M8402 t3171 nw960 vdd vdd pch w=2u l=180n
CT3174 t3174 0 0.1f
M8403 t3171 nw179 t3174 0 nch w=1u l=180n
M8404 t3174 nw960 0 0 nch w=1u l=180n
M8405 t3172 nw179 vdd vdd pch w=2u l=180n
M8406 t3172 t3171 vdd vdd pch w=2u l=180n
CT3175 t3175 0 0.1f
M8407 t3172 nw179 t3175 0 nch w=1u l=180n
M8408 t3175 t3171 0 0 nch w=1u l=180n
M8409 t3173 nw960 vdd vdd pch w=2u l=180n
M8410 t3173 t3171 vdd vdd pch w=2u l=180n
CT3176 t3176 0 0.1f
M8411 t3173 nw960 t3176 0 nch w=1u l=180n
M8412 t3176 t3171 0 0 nch w=1u l=180n
M8413 nw1031 t3172 vdd vdd pch w=2u l=180n
M8414 nw1031 t3173 vdd vdd pch w=2u l=180n
CT3177 t3177 0 0.1f
M8415 nw1031 t3172 t3177 0 nch w=1u l=180n
M8416 t3177 t3173 0 0 nch w=1u l=180n
Cnw1031 nw1031 0 2f
CT3178 t3178 0 0.1f
CT3179 t3179 0 0.1f
CT3180 t3180 0 0.1f
M8417 t3178 nw1031 vdd vdd pch w=2u l=180n
M8418 t3178 nw1030 vdd vdd pch w=2u l=180n
CT3181 t3181 0 0.1f
M8419 t3178 nw1031 t3181 0 nch w=1u l=180n
M8420 t3181 nw1030 0 0 nch w=1u l=180n
M8421 t3179 nw1031 vdd vdd pch w=2u l=180n
M8422 t3179 t3178 vdd vdd pch w=2u l=180n
CT3182 t3182 0 0.1f
M8423 t3179 nw1031 t3182 0 nch w=1u l=180n
M8424 t3182 t3178 0 0 nch w=1u l=180n
M8425 t3180 nw1030 vdd vdd pch w=2u l=180n
M8426 t3180 t3178 vdd vdd pch w=2u l=180n
CT3183 t3183 0 0.1f
M8427 t3180 nw1030 t3183 0 nch w=1u l=180n
M8428 t3183 t3178 0 0 nch w=1u l=180n
M8429 nw1032 t3179 vdd vdd pch w=2u l=180n
M8430 nw1032 t3180 vdd vdd pch w=2u l=180n
CT3184 t3184 0 0.1f
M8431 nw1032 t3179 t3184 0 nch w=1u l=180n
M8432 t3184 t3180 0 0 nch w=1u l=180n
Cnw1032 nw1032 0 2f
M8433 nw1033 nw179 vdd vdd pch w=2u l=180n
M8434 nw1033 nw960 vdd vdd pch w=2u l=180n
CT3185 t3185 0 0.1f
M8435 nw1033 nw179 t3185 0 nch w=1u l=180n
M8436 t3185 nw960 0 0 nch w=1u l=180n
Cnw1033 nw1033 0 2f
M8437 nw1034 nw1031 vdd vdd pch w=2u l=180n
M8438 nw1034 nw1030 vdd vdd pch w=2u l=180n
CT3186 t3186 0 0.1f
M8439 nw1034 nw1031 t3186 0 nch w=1u l=180n
M8440 t3186 nw1030 0 0 nch w=1u l=180n
Cnw1034 nw1034 0 2f
M8441 nw1035 nw1033 vdd vdd pch w=2u l=180n
M8442 nw1035 nw1034 vdd vdd pch w=2u l=180n
CT3187 t3187 0 0.1f
M8443 nw1035 nw1033 t3187 0 nch w=1u l=180n
M8444 t3187 nw1034 0 0 nch w=1u l=180n
Cnw1035 nw1035 0 2f
CT3188 t3188 0 0.1f
CT3189 t3189 0 0.1f
CT3190 t3190 0 0.1f
M8445 t3188 nw180 vdd vdd pch w=2u l=180n
M8446 t3188 nw965 vdd vdd pch w=2u l=180n
CT3191 t3191 0 0.1f
M8447 t3188 nw180 t3191 0 nch w=1u l=180n
M8448 t3191 nw965 0 0 nch w=1u l=180n
M8449 t3189 nw180 vdd vdd pch w=2u l=180n
M8450 t3189 t3188 vdd vdd pch w=2u l=180n
CT3192 t3192 0 0.1f
M8451 t3189 nw180 t3192 0 nch w=1u l=180n
M8452 t3192 t3188 0 0 nch w=1u l=180n
M8453 t3190 nw965 vdd vdd pch w=2u l=180n
M8454 t3190 t3188 vdd vdd pch w=2u l=180n
CT3193 t3193 0 0.1f
M8455 t3190 nw965 t3193 0 nch w=1u l=180n
M8456 t3193 t3188 0 0 nch w=1u l=180n
M8457 nw1036 t3189 vdd vdd pch w=2u l=180n
M8458 nw1036 t3190 vdd vdd pch w=2u l=180n
CT3194 t3194 0 0.1f
M8459 nw1036 t3189 t3194 0 nch w=1u l=180n
M8460 t3194 t3190 0 0 nch w=1u l=180n
Cnw1036 nw1036 0 2f
CT3195 t3195 0 0.1f
CT3196 t3196 0 0.1f
CT3197 t3197 0 0.1f
M8461 t3195 nw1036 vdd vdd pch w=2u l=180n
M8462 t3195 nw1035 vdd vdd pch w=2u l=180n
CT3198 t3198 0 0.1f
M8463 t3195 nw1036 t3198 0 nch w=1u l=180n
M8464 t3198 nw1035 0 0 nch w=1u l=180n
M8465 t3196 nw1036 vdd vdd pch w=2u l=180n
M8466 t3196 t3195 vdd vdd pch w=2u l=180n
CT3199 t3199 0 0.1f
M8467 t3196 nw1036 t3199 0 nch w=1u l=180n
M8468 t3199 t3195 0 0 nch w=1u l=180n
M8469 t3197 nw1035 vdd vdd pch w=2u l=180n
M8470 t3197 t3195 vdd vdd pch w=2u l=180n
CT3200 t3200 0 0.1f
M8471 t3197 nw1035 t3200 0 nch w=1u l=180n
M8472 t3200 t3195 0 0 nch w=1u l=180n
M8473 nw1037 t3196 vdd vdd pch w=2u l=180n
M8474 nw1037 t3197 vdd vdd pch w=2u l=180n
CT3201 t3201 0 0.1f
M8475 nw1037 t3196 t3201 0 nch w=1u l=180n
M8476 t3201 t3197 0 0 nch w=1u l=180n
Cnw1037 nw1037 0 2f
M8477 nw1038 nw180 vdd vdd pch w=2u l=180n
M8478 nw1038 nw965 vdd vdd pch w=2u l=180n
CT3202 t3202 0 0.1f
M8479 nw1038 nw180 t3202 0 nch w=1u l=180n
M8480 t3202 nw965 0 0 nch w=1u l=180n
Cnw1038 nw1038 0 2f
M8481 nw1039 nw1036 vdd vdd pch w=2u l=180n
M8482 nw1039 nw1035 vdd vdd pch w=2u l=180n
CT3203 t3203 0 0.1f
M8483 nw1039 nw1036 t3203 0 nch w=1u l=180n
M8484 t3203 nw1035 0 0 nch w=1u l=180n
Cnw1039 nw1039 0 2f
M8485 nw1040 nw1038 vdd vdd pch w=2u l=180n
M8486 nw1040 nw1039 vdd vdd pch w=2u l=180n
CT3204 t3204 0 0.1f
M8487 nw1040 nw1038 t3204 0 nch w=1u l=180n
M8488 t3204 nw1039 0 0 nch w=1u l=180n
Cnw1040 nw1040 0 2f
CT3205 t3205 0 0.1f
CT3206 t3206 0 0.1f
CT3207 t3207 0 0.1f
M8489 t3205 nw181 vdd vdd pch w=2u l=180n
M8490 t3205 nw970 vdd vdd pch w=2u l=180n
CT3208 t3208 0 0.1f
M8491 t3205 nw181 t3208 0 nch w=1u l=180n
M8492 t3208 nw970 0 0 nch w=1u l=180n
M8493 t3206 nw181 vdd vdd pch w=2u l=180n
M8494 t3206 t3205 vdd vdd pch w=2u l=180n
CT3209 t3209 0 0.1f
M8495 t3206 nw181 t3209 0 nch w=1u l=180n
M8496 t3209 t3205 0 0 nch w=1u l=180n
M8497 t3207 nw970 vdd vdd pch w=2u l=180n
M8498 t3207 t3205 vdd vdd pch w=2u l=180n
CT3210 t3210 0 0.1f
M8499 t3207 nw970 t3210 0 nch w=1u l=180n
M8500 t3210 t3205 0 0 nch w=1u l=180n
M8501 nw1041 t3206 vdd vdd pch w=2u l=180n
M8502 nw1041 t3207 vdd vdd pch w=2u l=180n
CT3211 t3211 0 0.1f
M8503 nw1041 t3206 t3211 0 nch w=1u l=180n
M8504 t3211 t3207 0 0 nch w=1u l=180n
Cnw1041 nw1041 0 2f
CT3212 t3212 0 0.1f
CT3213 t3213 0 0.1f
CT3214 t3214 0 0.1f
M8505 t3212 nw1041 vdd vdd pch w=2u l=180n
M8506 t3212 nw1040 vdd vdd pch w=2u l=180n
CT3215 t3215 0 0.1f
M8507 t3212 nw1041 t3215 0 nch w=1u l=180n
M8508 t3215 nw1040 0 0 nch w=1u l=180n
M8509 t3213 nw1041 vdd vdd pch w=2u l=180n
M8510 t3213 t3212 vdd vdd pch w=2u l=180n
CT3216 t3216 0 0.1f
M8511 t3213 nw1041 t3216 0 nch w=1u l=180n
M8512 t3216 t3212 0 0 nch w=1u l=180n
M8513 t3214 nw1040 vdd vdd pch w=2u l=180n
M8514 t3214 t3212 vdd vdd pch w=2u l=180n
CT3217 t3217 0 0.1f
M8515 t3214 nw1040 t3217 0 nch w=1u l=180n
M8516 t3217 t3212 0 0 nch w=1u l=180n
M8517 nw1042 t3213 vdd vdd pch w=2u l=180n
M8518 nw1042 t3214 vdd vdd pch w=2u l=180n
CT3218 t3218 0 0.1f
M8519 nw1042 t3213 t3218 0 nch w=1u l=180n
M8520 t3218 t3214 0 0 nch w=1u l=180n
Cnw1042 nw1042 0 2f
M8521 nw1043 nw181 vdd vdd pch w=2u l=180n
M8522 nw1043 nw970 vdd vdd pch w=2u l=180n
CT3219 t3219 0 0.1f
M8523 nw1043 nw181 t3219 0 nch w=1u l=180n
M8524 t3219 nw970 0 0 nch w=1u l=180n
Cnw1043 nw1043 0 2f
M8525 nw1044 nw1041 vdd vdd pch w=2u l=180n
M8526 nw1044 nw1040 vdd vdd pch w=2u l=180n
CT3220 t3220 0 0.1f
M8527 nw1044 nw1041 t3220 0 nch w=1u l=180n
M8528 t3220 nw1040 0 0 nch w=1u l=180n
Cnw1044 nw1044 0 2f
M8529 nw1045 nw1043 vdd vdd pch w=2u l=180n
M8530 nw1045 nw1044 vdd vdd pch w=2u l=180n
CT3221 t3221 0 0.1f
M8531 nw1045 nw1043 t3221 0 nch w=1u l=180n
M8532 t3221 nw1044 0 0 nch w=1u l=180n
Cnw1045 nw1045 0 2f
CT3222 t3222 0 0.1f
CT3223 t3223 0 0.1f
CT3224 t3224 0 0.1f
M8533 t3222 nw182 vdd vdd pch w=2u l=180n
M8534 t3222 nw975 vdd vdd pch w=2u l=180n
CT3225 t3225 0 0.1f
M8535 t3222 nw182 t3225 0 nch w=1u l=180n
M8536 t3225 nw975 0 0 nch w=1u l=180n
M8537 t3223 nw182 vdd vdd pch w=2u l=180n
M8538 t3223 t3222 vdd vdd pch w=2u l=180n
CT3226 t3226 0 0.1f
M8539 t3223 nw182 t3226 0 nch w=1u l=180n
M8540 t3226 t3222 0 0 nch w=1u l=180n
M8541 t3224 nw975 vdd vdd pch w=2u l=180n
M8542 t3224 t3222 vdd vdd pch w=2u l=180n
CT3227 t3227 0 0.1f
M8543 t3224 nw975 t3227 0 nch w=1u l=180n
M8544 t3227 t3222 0 0 nch w=1u l=180n
M8545 nw1046 t3223 vdd vdd pch w=2u l=180n
M8546 nw1046 t3224 vdd vdd pch w=2u l=180n
CT3228 t3228 0 0.1f
M8547 nw1046 t3223 t3228 0 nch w=1u l=180n
M8548 t3228 t3224 0 0 nch w=1u l=180n
Cnw1046 nw1046 0 2f
CT3229 t3229 0 0.1f
CT3230 t3230 0 0.1f
CT3231 t3231 0 0.1f
M8549 t3229 nw1046 vdd vdd pch w=2u l=180n
M8550 t3229 nw1045 vdd vdd pch w=2u l=180n
CT3232 t3232 0 0.1f
M8551 t3229 nw1046 t3232 0 nch w=1u l=180n
M8552 t3232 nw1045 0 0 nch w=1u l=180n
M8553 t3230 nw1046 vdd vdd pch w=2u l=180n
M8554 t3230 t3229 vdd vdd pch w=2u l=180n
CT3233 t3233 0 0.1f
M8555 t3230 nw1046 t3233 0 nch w=1u l=180n
M8556 t3233 t3229 0 0 nch w=1u l=180n
M8557 t3231 nw1045 vdd vdd pch w=2u l=180n
M8558 t3231 t3229 vdd vdd pch w=2u l=180n
CT3234 t3234 0 0.1f
M8559 t3231 nw1045 t3234 0 nch w=1u l=180n
M8560 t3234 t3229 0 0 nch w=1u l=180n
M8561 nw1047 t3230 vdd vdd pch w=2u l=180n
M8562 nw1047 t3231 vdd vdd pch w=2u l=180n
CT3235 t3235 0 0.1f
M8563 nw1047 t3230 t3235 0 nch w=1u l=180n
M8564 t3235 t3231 0 0 nch w=1u l=180n
Cnw1047 nw1047 0 2f
M8565 nw1048 nw182 vdd vdd pch w=2u l=180n
M8566 nw1048 nw975 vdd vdd pch w=2u l=180n
CT3236 t3236 0 0.1f
M8567 nw1048 nw182 t3236 0 nch w=1u l=180n
M8568 t3236 nw975 0 0 nch w=1u l=180n
Cnw1048 nw1048 0 2f
M8569 nw1049 nw1046 vdd vdd pch w=2u l=180n
M8570 nw1049 nw1045 vdd vdd pch w=2u l=180n
CT3237 t3237 0 0.1f
M8571 nw1049 nw1046 t3237 0 nch w=1u l=180n
M8572 t3237 nw1045 0 0 nch w=1u l=180n
Cnw1049 nw1049 0 2f
M8573 nw1050 nw1048 vdd vdd pch w=2u l=180n
M8574 nw1050 nw1049 vdd vdd pch w=2u l=180n
CT3238 t3238 0 0.1f
M8575 nw1050 nw1048 t3238 0 nch w=1u l=180n
M8576 t3238 nw1049 0 0 nch w=1u l=180n
Cnw1050 nw1050 0 2f
CT3239 t3239 0 0.1f
CT3240 t3240 0 0.1f
CT3241 t3241 0 0.1f
M8577 t3239 nw183 vdd vdd pch w=2u l=180n
M8578 t3239 nw980 vdd vdd pch w=2u l=180n
CT3242 t3242 0 0.1f
M8579 t3239 nw183 t3242 0 nch w=1u l=180n
M8580 t3242 nw980 0 0 nch w=1u l=180n
M8581 t3240 nw183 vdd vdd pch w=2u l=180n
M8582 t3240 t3239 vdd vdd pch w=2u l=180n
CT3243 t3243 0 0.1f
M8583 t3240 nw183 t3243 0 nch w=1u l=180n
M8584 t3243 t3239 0 0 nch w=1u l=180n
M8585 t3241 nw980 vdd vdd pch w=2u l=180n
M8586 t3241 t3239 vdd vdd pch w=2u l=180n
CT3244 t3244 0 0.1f
M8587 t3241 nw980 t3244 0 nch w=1u l=180n
M8588 t3244 t3239 0 0 nch w=1u l=180n
M8589 nw1051 t3240 vdd vdd pch w=2u l=180n
M8590 nw1051 t3241 vdd vdd pch w=2u l=180n
CT3245 t3245 0 0.1f
M8591 nw1051 t3240 t3245 0 nch w=1u l=180n
M8592 t3245 t3241 0 0 nch w=1u l=180n
Cnw1051 nw1051 0 2f
CT3246 t3246 0 0.1f
CT3247 t3247 0 0.1f
CT3248 t3248 0 0.1f
M8593 t3246 nw1051 vdd vdd pch w=2u l=180n
M8594 t3246 nw1050 vdd vdd pch w=2u l=180n
CT3249 t3249 0 0.1f
M8595 t3246 nw1051 t3249 0 nch w=1u l=180n
M8596 t3249 nw1050 0 0 nch w=1u l=180n
M8597 t3247 nw1051 vdd vdd pch w=2u l=180n
M8598 t3247 t3246 vdd vdd pch w=2u l=180n
CT3250 t3250 0 0.1f
M8599 t3247 nw1051 t3250 0 nch w=1u l=180n
M8600 t3250 t3246 0 0 nch w=1u l=180n
M8601 t3248 nw1050 vdd vdd pch w=2u l=180n
M8602 t3248 t3246 vdd vdd pch w=2u l=180n
CT3251 t3251 0 0.1f
M8603 t3248 nw1050 t3251 0 nch w=1u l=180n
M8604 t3251 t3246 0 0 nch w=1u l=180n
M8605 nw1052 t3247 vdd vdd pch w=2u l=180n
M8606 nw1052 t3248 vdd vdd pch w=2u l=180n
CT3252 t3252 0 0.1f
M8607 nw1052 t3247 t3252 0 nch w=1u l=180n
M8608 t3252 t3248 0 0 nch w=1u l=180n
Cnw1052 nw1052 0 2f
M8609 nw1053 nw183 vdd vdd pch w=2u l=180n
M8610 nw1053 nw980 vdd vdd pch w=2u l=180n
CT3253 t3253 0 0.1f
M8611 nw1053 nw183 t3253 0 nch w=1u l=180n
M8612 t3253 nw980 0 0 nch w=1u l=180n
Cnw1053 nw1053 0 2f
M8613 nw1054 nw1051 vdd vdd pch w=2u l=180n
M8614 nw1054 nw1050 vdd vdd pch w=2u l=180n
CT3254 t3254 0 0.1f
M8615 nw1054 nw1051 t3254 0 nch w=1u l=180n
M8616 t3254 nw1050 0 0 nch w=1u l=180n
Cnw1054 nw1054 0 2f
M8617 nw1055 nw1053 vdd vdd pch w=2u l=180n
M8618 nw1055 nw1054 vdd vdd pch w=2u l=180n
CT3255 t3255 0 0.1f
M8619 nw1055 nw1053 t3255 0 nch w=1u l=180n
M8620 t3255 nw1054 0 0 nch w=1u l=180n
Cnw1055 nw1055 0 2f
CT3256 t3256 0 0.1f
CT3257 t3257 0 0.1f
CT3258 t3258 0 0.1f
M8621 t3256 nw184 vdd vdd pch w=2u l=180n
M8622 t3256 nw985 vdd vdd pch w=2u l=180n
CT3259 t3259 0 0.1f
M8623 t3256 nw184 t3259 0 nch w=1u l=180n
M8624 t3259 nw985 0 0 nch w=1u l=180n
M8625 t3257 nw184 vdd vdd pch w=2u l=180n
M8626 t3257 t3256 vdd vdd pch w=2u l=180n
CT3260 t3260 0 0.1f
M8627 t3257 nw184 t3260 0 nch w=1u l=180n
M8628 t3260 t3256 0 0 nch w=1u l=180n
M8629 t3258 nw985 vdd vdd pch w=2u l=180n
M8630 t3258 t3256 vdd vdd pch w=2u l=180n
CT3261 t3261 0 0.1f
M8631 t3258 nw985 t3261 0 nch w=1u l=180n
M8632 t3261 t3256 0 0 nch w=1u l=180n
M8633 nw1056 t3257 vdd vdd pch w=2u l=180n
M8634 nw1056 t3258 vdd vdd pch w=2u l=180n
CT3262 t3262 0 0.1f
M8635 nw1056 t3257 t3262 0 nch w=1u l=180n
M8636 t3262 t3258 0 0 nch w=1u l=180n
Cnw1056 nw1056 0 2f
CT3263 t3263 0 0.1f
CT3264 t3264 0 0.1f
CT3265 t3265 0 0.1f
M8637 t3263 nw1056 vdd vdd pch w=2u l=180n
M8638 t3263 nw1055 vdd vdd pch w=2u l=180n
CT3266 t3266 0 0.1f
M8639 t3263 nw1056 t3266 0 nch w=1u l=180n
M8640 t3266 nw1055 0 0 nch w=1u l=180n
M8641 t3264 nw1056 vdd vdd pch w=2u l=180n
M8642 t3264 t3263 vdd vdd pch w=2u l=180n
CT3267 t3267 0 0.1f
M8643 t3264 nw1056 t3267 0 nch w=1u l=180n
M8644 t3267 t3263 0 0 nch w=1u l=180n
M8645 t3265 nw1055 vdd vdd pch w=2u l=180n
M8646 t3265 t3263 vdd vdd pch w=2u l=180n
CT3268 t3268 0 0.1f
M8647 t3265 nw1055 t3268 0 nch w=1u l=180n
M8648 t3268 t3263 0 0 nch w=1u l=180n
M8649 nw1057 t3264 vdd vdd pch w=2u l=180n
M8650 nw1057 t3265 vdd vdd pch w=2u l=180n
CT3269 t3269 0 0.1f
M8651 nw1057 t3264 t3269 0 nch w=1u l=180n
M8652 t3269 t3265 0 0 nch w=1u l=180n
Cnw1057 nw1057 0 2f
M8653 nw1058 nw184 vdd vdd pch w=2u l=180n
M8654 nw1058 nw985 vdd vdd pch w=2u l=180n
CT3270 t3270 0 0.1f
M8655 nw1058 nw184 t3270 0 nch w=1u l=180n
M8656 t3270 nw985 0 0 nch w=1u l=180n
Cnw1058 nw1058 0 2f
M8657 nw1059 nw1056 vdd vdd pch w=2u l=180n
M8658 nw1059 nw1055 vdd vdd pch w=2u l=180n
CT3271 t3271 0 0.1f
M8659 nw1059 nw1056 t3271 0 nch w=1u l=180n
M8660 t3271 nw1055 0 0 nch w=1u l=180n
Cnw1059 nw1059 0 2f
M8661 nw1060 nw1058 vdd vdd pch w=2u l=180n
M8662 nw1060 nw1059 vdd vdd pch w=2u l=180n
CT3272 t3272 0 0.1f
M8663 nw1060 nw1058 t3272 0 nch w=1u l=180n
M8664 t3272 nw1059 0 0 nch w=1u l=180n
Cnw1060 nw1060 0 2f
CT3273 t3273 0 0.1f
CT3274 t3274 0 0.1f
CT3275 t3275 0 0.1f
M8665 t3273 nw185 vdd vdd pch w=2u l=180n
M8666 t3273 nw990 vdd vdd pch w=2u l=180n
CT3276 t3276 0 0.1f
M8667 t3273 nw185 t3276 0 nch w=1u l=180n
M8668 t3276 nw990 0 0 nch w=1u l=180n
M8669 t3274 nw185 vdd vdd pch w=2u l=180n
M8670 t3274 t3273 vdd vdd pch w=2u l=180n
CT3277 t3277 0 0.1f
M8671 t3274 nw185 t3277 0 nch w=1u l=180n
M8672 t3277 t3273 0 0 nch w=1u l=180n
M8673 t3275 nw990 vdd vdd pch w=2u l=180n
M8674 t3275 t3273 vdd vdd pch w=2u l=180n
CT3278 t3278 0 0.1f
M8675 t3275 nw990 t3278 0 nch w=1u l=180n
M8676 t3278 t3273 0 0 nch w=1u l=180n
M8677 nw1061 t3274 vdd vdd pch w=2u l=180n
M8678 nw1061 t3275 vdd vdd pch w=2u l=180n
CT3279 t3279 0 0.1f
M8679 nw1061 t3274 t3279 0 nch w=1u l=180n
M8680 t3279 t3275 0 0 nch w=1u l=180n
Cnw1061 nw1061 0 2f
CT3280 t3280 0 0.1f
CT3281 t3281 0 0.1f
CT3282 t3282 0 0.1f
M8681 t3280 nw1061 vdd vdd pch w=2u l=180n
M8682 t3280 nw1060 vdd vdd pch w=2u l=180n
CT3283 t3283 0 0.1f
M8683 t3280 nw1061 t3283 0 nch w=1u l=180n
M8684 t3283 nw1060 0 0 nch w=1u l=180n
M8685 t3281 nw1061 vdd vdd pch w=2u l=180n
M8686 t3281 t3280 vdd vdd pch w=2u l=180n
CT3284 t3284 0 0.1f
M8687 t3281 nw1061 t3284 0 nch w=1u l=180n
M8688 t3284 t3280 0 0 nch w=1u l=180n
M8689 t3282 nw1060 vdd vdd pch w=2u l=180n
M8690 t3282 t3280 vdd vdd pch w=2u l=180n
CT3285 t3285 0 0.1f
M8691 t3282 nw1060 t3285 0 nch w=1u l=180n
M8692 t3285 t3280 0 0 nch w=1u l=180n
M8693 nw1062 t3281 vdd vdd pch w=2u l=180n
M8694 nw1062 t3282 vdd vdd pch w=2u l=180n
CT3286 t3286 0 0.1f
M8695 nw1062 t3281 t3286 0 nch w=1u l=180n
M8696 t3286 t3282 0 0 nch w=1u l=180n
Cnw1062 nw1062 0 2f
M8697 nw1063 nw185 vdd vdd pch w=2u l=180n
M8698 nw1063 nw990 vdd vdd pch w=2u l=180n
CT3287 t3287 0 0.1f
M8699 nw1063 nw185 t3287 0 nch w=1u l=180n
M8700 t3287 nw990 0 0 nch w=1u l=180n
Cnw1063 nw1063 0 2f
M8701 nw1064 nw1061 vdd vdd pch w=2u l=180n
M8702 nw1064 nw1060 vdd vdd pch w=2u l=180n
CT3288 t3288 0 0.1f
M8703 nw1064 nw1061 t3288 0 nch w=1u l=180n
M8704 t3288 nw1060 0 0 nch w=1u l=180n
Cnw1064 nw1064 0 2f
M8705 nw1065 nw1063 vdd vdd pch w=2u l=180n
M8706 nw1065 nw1064 vdd vdd pch w=2u l=180n
CT3289 t3289 0 0.1f
M8707 nw1065 nw1063 t3289 0 nch w=1u l=180n
M8708 t3289 nw1064 0 0 nch w=1u l=180n
Cnw1065 nw1065 0 2f
CT3290 t3290 0 0.1f
CT3291 t3291 0 0.1f
CT3292 t3292 0 0.1f
M8709 t3290 nw186 vdd vdd pch w=2u l=180n
M8710 t3290 nw995 vdd vdd pch w=2u l=180n
CT3293 t3293 0 0.1f
M8711 t3290 nw186 t3293 0 nch w=1u l=180n
M8712 t3293 nw995 0 0 nch w=1u l=180n
M8713 t3291 nw186 vdd vdd pch w=2u l=180n
M8714 t3291 t3290 vdd vdd pch w=2u l=180n
CT3294 t3294 0 0.1f
M8715 t3291 nw186 t3294 0 nch w=1u l=180n
M8716 t3294 t3290 0 0 nch w=1u l=180n
M8717 t3292 nw995 vdd vdd pch w=2u l=180n
M8718 t3292 t3290 vdd vdd pch w=2u l=180n
CT3295 t3295 0 0.1f
M8719 t3292 nw995 t3295 0 nch w=1u l=180n
M8720 t3295 t3290 0 0 nch w=1u l=180n
M8721 nw1066 t3291 vdd vdd pch w=2u l=180n
M8722 nw1066 t3292 vdd vdd pch w=2u l=180n
CT3296 t3296 0 0.1f
M8723 nw1066 t3291 t3296 0 nch w=1u l=180n
M8724 t3296 t3292 0 0 nch w=1u l=180n
Cnw1066 nw1066 0 2f
CT3297 t3297 0 0.1f
CT3298 t3298 0 0.1f
CT3299 t3299 0 0.1f
M8725 t3297 nw1066 vdd vdd pch w=2u l=180n
M8726 t3297 nw1065 vdd vdd pch w=2u l=180n
CT3300 t3300 0 0.1f
M8727 t3297 nw1066 t3300 0 nch w=1u l=180n
M8728 t3300 nw1065 0 0 nch w=1u l=180n
M8729 t3298 nw1066 vdd vdd pch w=2u l=180n
M8730 t3298 t3297 vdd vdd pch w=2u l=180n
CT3301 t3301 0 0.1f
M8731 t3298 nw1066 t3301 0 nch w=1u l=180n
M8732 t3301 t3297 0 0 nch w=1u l=180n
M8733 t3299 nw1065 vdd vdd pch w=2u l=180n
M8734 t3299 t3297 vdd vdd pch w=2u l=180n
CT3302 t3302 0 0.1f
M8735 t3299 nw1065 t3302 0 nch w=1u l=180n
M8736 t3302 t3297 0 0 nch w=1u l=180n
M8737 nw1067 t3298 vdd vdd pch w=2u l=180n
M8738 nw1067 t3299 vdd vdd pch w=2u l=180n
CT3303 t3303 0 0.1f
M8739 nw1067 t3298 t3303 0 nch w=1u l=180n
M8740 t3303 t3299 0 0 nch w=1u l=180n
Cnw1067 nw1067 0 2f
M8741 nw1068 nw186 vdd vdd pch w=2u l=180n
M8742 nw1068 nw995 vdd vdd pch w=2u l=180n
CT3304 t3304 0 0.1f
M8743 nw1068 nw186 t3304 0 nch w=1u l=180n
M8744 t3304 nw995 0 0 nch w=1u l=180n
Cnw1068 nw1068 0 2f
M8745 nw1069 nw1066 vdd vdd pch w=2u l=180n
M8746 nw1069 nw1065 vdd vdd pch w=2u l=180n
CT3305 t3305 0 0.1f
M8747 nw1069 nw1066 t3305 0 nch w=1u l=180n
M8748 t3305 nw1065 0 0 nch w=1u l=180n
Cnw1069 nw1069 0 2f
M8749 nw1070 nw1068 vdd vdd pch w=2u l=180n
M8750 nw1070 nw1069 vdd vdd pch w=2u l=180n
CT3306 t3306 0 0.1f
M8751 nw1070 nw1068 t3306 0 nch w=1u l=180n
M8752 t3306 nw1069 0 0 nch w=1u l=180n
Cnw1070 nw1070 0 2f
CT3307 t3307 0 0.1f
CT3308 t3308 0 0.1f
CT3309 t3309 0 0.1f
M8753 t3307 nw187 vdd vdd pch w=2u l=180n
M8754 t3307 nw1000 vdd vdd pch w=2u l=180n
CT3310 t3310 0 0.1f
M8755 t3307 nw187 t3310 0 nch w=1u l=180n
M8756 t3310 nw1000 0 0 nch w=1u l=180n
M8757 t3308 nw187 vdd vdd pch w=2u l=180n
M8758 t3308 t3307 vdd vdd pch w=2u l=180n
CT3311 t3311 0 0.1f
M8759 t3308 nw187 t3311 0 nch w=1u l=180n
M8760 t3311 t3307 0 0 nch w=1u l=180n
M8761 t3309 nw1000 vdd vdd pch w=2u l=180n
M8762 t3309 t3307 vdd vdd pch w=2u l=180n
CT3312 t3312 0 0.1f
M8763 t3309 nw1000 t3312 0 nch w=1u l=180n
M8764 t3312 t3307 0 0 nch w=1u l=180n
M8765 nw1071 t3308 vdd vdd pch w=2u l=180n
M8766 nw1071 t3309 vdd vdd pch w=2u l=180n
CT3313 t3313 0 0.1f
M8767 nw1071 t3308 t3313 0 nch w=1u l=180n
M8768 t3313 t3309 0 0 nch w=1u l=180n
Cnw1071 nw1071 0 2f
CT3314 t3314 0 0.1f
CT3315 t3315 0 0.1f
CT3316 t3316 0 0.1f
M8769 t3314 nw1071 vdd vdd pch w=2u l=180n
M8770 t3314 nw1070 vdd vdd pch w=2u l=180n
CT3317 t3317 0 0.1f
M8771 t3314 nw1071 t3317 0 nch w=1u l=180n
M8772 t3317 nw1070 0 0 nch w=1u l=180n
M8773 t3315 nw1071 vdd vdd pch w=2u l=180n
M8774 t3315 t3314 vdd vdd pch w=2u l=180n
CT3318 t3318 0 0.1f
M8775 t3315 nw1071 t3318 0 nch w=1u l=180n
M8776 t3318 t3314 0 0 nch w=1u l=180n
M8777 t3316 nw1070 vdd vdd pch w=2u l=180n
M8778 t3316 t3314 vdd vdd pch w=2u l=180n
CT3319 t3319 0 0.1f
M8779 t3316 nw1070 t3319 0 nch w=1u l=180n
M8780 t3319 t3314 0 0 nch w=1u l=180n
M8781 nw1072 t3315 vdd vdd pch w=2u l=180n
M8782 nw1072 t3316 vdd vdd pch w=2u l=180n
CT3320 t3320 0 0.1f
M8783 nw1072 t3315 t3320 0 nch w=1u l=180n
M8784 t3320 t3316 0 0 nch w=1u l=180n
Cnw1072 nw1072 0 2f
M8785 nw1073 nw187 vdd vdd pch w=2u l=180n
M8786 nw1073 nw1000 vdd vdd pch w=2u l=180n
CT3321 t3321 0 0.1f
M8787 nw1073 nw187 t3321 0 nch w=1u l=180n
M8788 t3321 nw1000 0 0 nch w=1u l=180n
Cnw1073 nw1073 0 2f
M8789 nw1074 nw1071 vdd vdd pch w=2u l=180n
M8790 nw1074 nw1070 vdd vdd pch w=2u l=180n
CT3322 t3322 0 0.1f
M8791 nw1074 nw1071 t3322 0 nch w=1u l=180n
M8792 t3322 nw1070 0 0 nch w=1u l=180n
Cnw1074 nw1074 0 2f
M8793 nw1075 nw1073 vdd vdd pch w=2u l=180n
M8794 nw1075 nw1074 vdd vdd pch w=2u l=180n
CT3323 t3323 0 0.1f
M8795 nw1075 nw1073 t3323 0 nch w=1u l=180n
M8796 t3323 nw1074 0 0 nch w=1u l=180n
Cnw1075 nw1075 0 2f
CT3324 t3324 0 0.1f
CT3325 t3325 0 0.1f
CT3326 t3326 0 0.1f
M8797 t3324 nw188 vdd vdd pch w=2u l=180n
M8798 t3324 nw1005 vdd vdd pch w=2u l=180n
CT3327 t3327 0 0.1f
M8799 t3324 nw188 t3327 0 nch w=1u l=180n
M8800 t3327 nw1005 0 0 nch w=1u l=180n
M8801 t3325 nw188 vdd vdd pch w=2u l=180n
M8802 t3325 t3324 vdd vdd pch w=2u l=180n
CT3328 t3328 0 0.1f
M8803 t3325 nw188 t3328 0 nch w=1u l=180n
M8804 t3328 t3324 0 0 nch w=1u l=180n
M8805 t3326 nw1005 vdd vdd pch w=2u l=180n
M8806 t3326 t3324 vdd vdd pch w=2u l=180n
CT3329 t3329 0 0.1f
M8807 t3326 nw1005 t3329 0 nch w=1u l=180n
M8808 t3329 t3324 0 0 nch w=1u l=180n
M8809 nw1076 t3325 vdd vdd pch w=2u l=180n
M8810 nw1076 t3326 vdd vdd pch w=2u l=180n
CT3330 t3330 0 0.1f
M8811 nw1076 t3325 t3330 0 nch w=1u l=180n
M8812 t3330 t3326 0 0 nch w=1u l=180n
Cnw1076 nw1076 0 2f
CT3331 t3331 0 0.1f
CT3332 t3332 0 0.1f
CT3333 t3333 0 0.1f
M8813 t3331 nw1076 vdd vdd pch w=2u l=180n
M8814 t3331 nw1075 vdd vdd pch w=2u l=180n
CT3334 t3334 0 0.1f
M8815 t3331 nw1076 t3334 0 nch w=1u l=180n
M8816 t3334 nw1075 0 0 nch w=1u l=180n
M8817 t3332 nw1076 vdd vdd pch w=2u l=180n
M8818 t3332 t3331 vdd vdd pch w=2u l=180n
CT3335 t3335 0 0.1f
M8819 t3332 nw1076 t3335 0 nch w=1u l=180n
M8820 t3335 t3331 0 0 nch w=1u l=180n
M8821 t3333 nw1075 vdd vdd pch w=2u l=180n
M8822 t3333 t3331 vdd vdd pch w=2u l=180n
CT3336 t3336 0 0.1f
M8823 t3333 nw1075 t3336 0 nch w=1u l=180n
M8824 t3336 t3331 0 0 nch w=1u l=180n
M8825 nw1077 t3332 vdd vdd pch w=2u l=180n
M8826 nw1077 t3333 vdd vdd pch w=2u l=180n
CT3337 t3337 0 0.1f
M8827 nw1077 t3332 t3337 0 nch w=1u l=180n
M8828 t3337 t3333 0 0 nch w=1u l=180n
Cnw1077 nw1077 0 2f
M8829 nw1078 nw188 vdd vdd pch w=2u l=180n
M8830 nw1078 nw1005 vdd vdd pch w=2u l=180n
CT3338 t3338 0 0.1f
M8831 nw1078 nw188 t3338 0 nch w=1u l=180n
M8832 t3338 nw1005 0 0 nch w=1u l=180n
Cnw1078 nw1078 0 2f
M8833 nw1079 nw1076 vdd vdd pch w=2u l=180n
M8834 nw1079 nw1075 vdd vdd pch w=2u l=180n
CT3339 t3339 0 0.1f
M8835 nw1079 nw1076 t3339 0 nch w=1u l=180n
M8836 t3339 nw1075 0 0 nch w=1u l=180n
Cnw1079 nw1079 0 2f
M8837 nw1080 nw1078 vdd vdd pch w=2u l=180n
M8838 nw1080 nw1079 vdd vdd pch w=2u l=180n
CT3340 t3340 0 0.1f
M8839 nw1080 nw1078 t3340 0 nch w=1u l=180n
M8840 t3340 nw1079 0 0 nch w=1u l=180n
Cnw1080 nw1080 0 2f
CT3341 t3341 0 0.1f
CT3342 t3342 0 0.1f
CT3343 t3343 0 0.1f
M8841 t3341 nw189 vdd vdd pch w=2u l=180n
M8842 t3341 nw1010 vdd vdd pch w=2u l=180n
CT3344 t3344 0 0.1f
M8843 t3341 nw189 t3344 0 nch w=1u l=180n
M8844 t3344 nw1010 0 0 nch w=1u l=180n
M8845 t3342 nw189 vdd vdd pch w=2u l=180n
M8846 t3342 t3341 vdd vdd pch w=2u l=180n
CT3345 t3345 0 0.1f
M8847 t3342 nw189 t3345 0 nch w=1u l=180n
M8848 t3345 t3341 0 0 nch w=1u l=180n
M8849 t3343 nw1010 vdd vdd pch w=2u l=180n
M8850 t3343 t3341 vdd vdd pch w=2u l=180n
CT3346 t3346 0 0.1f
M8851 t3343 nw1010 t3346 0 nch w=1u l=180n
M8852 t3346 t3341 0 0 nch w=1u l=180n
M8853 nw1081 t3342 vdd vdd pch w=2u l=180n
M8854 nw1081 t3343 vdd vdd pch w=2u l=180n
CT3347 t3347 0 0.1f
M8855 nw1081 t3342 t3347 0 nch w=1u l=180n
M8856 t3347 t3343 0 0 nch w=1u l=180n
Cnw1081 nw1081 0 2f
CT3348 t3348 0 0.1f
CT3349 t3349 0 0.1f
CT3350 t3350 0 0.1f
M8857 t3348 nw1081 vdd vdd pch w=2u l=180n
M8858 t3348 nw1080 vdd vdd pch w=2u l=180n
CT3351 t3351 0 0.1f
M8859 t3348 nw1081 t3351 0 nch w=1u l=180n
M8860 t3351 nw1080 0 0 nch w=1u l=180n
M8861 t3349 nw1081 vdd vdd pch w=2u l=180n
M8862 t3349 t3348 vdd vdd pch w=2u l=180n
CT3352 t3352 0 0.1f
M8863 t3349 nw1081 t3352 0 nch w=1u l=180n
M8864 t3352 t3348 0 0 nch w=1u l=180n
M8865 t3350 nw1080 vdd vdd pch w=2u l=180n
M8866 t3350 t3348 vdd vdd pch w=2u l=180n
CT3353 t3353 0 0.1f
M8867 t3350 nw1080 t3353 0 nch w=1u l=180n
M8868 t3353 t3348 0 0 nch w=1u l=180n
M8869 nw1082 t3349 vdd vdd pch w=2u l=180n
M8870 nw1082 t3350 vdd vdd pch w=2u l=180n
CT3354 t3354 0 0.1f
M8871 nw1082 t3349 t3354 0 nch w=1u l=180n
M8872 t3354 t3350 0 0 nch w=1u l=180n
Cnw1082 nw1082 0 2f
M8873 nw1083 nw189 vdd vdd pch w=2u l=180n
M8874 nw1083 nw1010 vdd vdd pch w=2u l=180n
CT3355 t3355 0 0.1f
M8875 nw1083 nw189 t3355 0 nch w=1u l=180n
M8876 t3355 nw1010 0 0 nch w=1u l=180n
Cnw1083 nw1083 0 2f
M8877 nw1084 nw1081 vdd vdd pch w=2u l=180n
M8878 nw1084 nw1080 vdd vdd pch w=2u l=180n
CT3356 t3356 0 0.1f
M8879 nw1084 nw1081 t3356 0 nch w=1u l=180n
M8880 t3356 nw1080 0 0 nch w=1u l=180n
Cnw1084 nw1084 0 2f
M8881 nw1085 nw1083 vdd vdd pch w=2u l=180n
M8882 nw1085 nw1084 vdd vdd pch w=2u l=180n
CT3357 t3357 0 0.1f
M8883 nw1085 nw1083 t3357 0 nch w=1u l=180n
M8884 t3357 nw1084 0 0 nch w=1u l=180n
Cnw1085 nw1085 0 2f
CT3358 t3358 0 0.1f
CT3359 t3359 0 0.1f
CT3360 t3360 0 0.1f
M8885 t3358 nw190 vdd vdd pch w=2u l=180n
M8886 t3358 nw1015 vdd vdd pch w=2u l=180n
CT3361 t3361 0 0.1f
M8887 t3358 nw190 t3361 0 nch w=1u l=180n
M8888 t3361 nw1015 0 0 nch w=1u l=180n
M8889 t3359 nw190 vdd vdd pch w=2u l=180n
M8890 t3359 t3358 vdd vdd pch w=2u l=180n
CT3362 t3362 0 0.1f
M8891 t3359 nw190 t3362 0 nch w=1u l=180n
M8892 t3362 t3358 0 0 nch w=1u l=180n
M8893 t3360 nw1015 vdd vdd pch w=2u l=180n
M8894 t3360 t3358 vdd vdd pch w=2u l=180n
CT3363 t3363 0 0.1f
M8895 t3360 nw1015 t3363 0 nch w=1u l=180n
M8896 t3363 t3358 0 0 nch w=1u l=180n
M8897 nw1086 t3359 vdd vdd pch w=2u l=180n
M8898 nw1086 t3360 vdd vdd pch w=2u l=180n
CT3364 t3364 0 0.1f
M8899 nw1086 t3359 t3364 0 nch w=1u l=180n
M8900 t3364 t3360 0 0 nch w=1u l=180n
Cnw1086 nw1086 0 2f
CT3365 t3365 0 0.1f
CT3366 t3366 0 0.1f
CT3367 t3367 0 0.1f
M8901 t3365 nw1086 vdd vdd pch w=2u l=180n
M8902 t3365 nw1085 vdd vdd pch w=2u l=180n
CT3368 t3368 0 0.1f
M8903 t3365 nw1086 t3368 0 nch w=1u l=180n
M8904 t3368 nw1085 0 0 nch w=1u l=180n
M8905 t3366 nw1086 vdd vdd pch w=2u l=180n
M8906 t3366 t3365 vdd vdd pch w=2u l=180n
CT3369 t3369 0 0.1f
M8907 t3366 nw1086 t3369 0 nch w=1u l=180n
M8908 t3369 t3365 0 0 nch w=1u l=180n
M8909 t3367 nw1085 vdd vdd pch w=2u l=180n
M8910 t3367 t3365 vdd vdd pch w=2u l=180n
CT3370 t3370 0 0.1f
M8911 t3367 nw1085 t3370 0 nch w=1u l=180n
M8912 t3370 t3365 0 0 nch w=1u l=180n
M8913 nw1087 t3366 vdd vdd pch w=2u l=180n
M8914 nw1087 t3367 vdd vdd pch w=2u l=180n
CT3371 t3371 0 0.1f
M8915 nw1087 t3366 t3371 0 nch w=1u l=180n
M8916 t3371 t3367 0 0 nch w=1u l=180n
Cnw1087 nw1087 0 2f
M8917 nw1088 nw190 vdd vdd pch w=2u l=180n
M8918 nw1088 nw1015 vdd vdd pch w=2u l=180n
CT3372 t3372 0 0.1f
M8919 nw1088 nw190 t3372 0 nch w=1u l=180n
M8920 t3372 nw1015 0 0 nch w=1u l=180n
Cnw1088 nw1088 0 2f
M8921 nw1089 nw1086 vdd vdd pch w=2u l=180n
M8922 nw1089 nw1085 vdd vdd pch w=2u l=180n
CT3373 t3373 0 0.1f
M8923 nw1089 nw1086 t3373 0 nch w=1u l=180n
M8924 t3373 nw1085 0 0 nch w=1u l=180n
Cnw1089 nw1089 0 2f
M8925 nw1090 nw1088 vdd vdd pch w=2u l=180n
M8926 nw1090 nw1089 vdd vdd pch w=2u l=180n
CT3374 t3374 0 0.1f
M8927 nw1090 nw1088 t3374 0 nch w=1u l=180n
M8928 t3374 nw1089 0 0 nch w=1u l=180n
Cnw1090 nw1090 0 2f
CT3375 t3375 0 0.1f
CT3376 t3376 0 0.1f
CT3377 t3377 0 0.1f
M8929 t3375 nw191 vdd vdd pch w=2u l=180n
M8930 t3375 nw1020 vdd vdd pch w=2u l=180n
CT3378 t3378 0 0.1f
M8931 t3375 nw191 t3378 0 nch w=1u l=180n
M8932 t3378 nw1020 0 0 nch w=1u l=180n
M8933 t3376 nw191 vdd vdd pch w=2u l=180n
M8934 t3376 t3375 vdd vdd pch w=2u l=180n
CT3379 t3379 0 0.1f
M8935 t3376 nw191 t3379 0 nch w=1u l=180n
M8936 t3379 t3375 0 0 nch w=1u l=180n
M8937 t3377 nw1020 vdd vdd pch w=2u l=180n
M8938 t3377 t3375 vdd vdd pch w=2u l=180n
CT3380 t3380 0 0.1f
M8939 t3377 nw1020 t3380 0 nch w=1u l=180n
M8940 t3380 t3375 0 0 nch w=1u l=180n
M8941 nw1091 t3376 vdd vdd pch w=2u l=180n
M8942 nw1091 t3377 vdd vdd pch w=2u l=180n
CT3381 t3381 0 0.1f
M8943 nw1091 t3376 t3381 0 nch w=1u l=180n
M8944 t3381 t3377 0 0 nch w=1u l=180n
Cnw1091 nw1091 0 2f
CT3382 t3382 0 0.1f
CT3383 t3383 0 0.1f
CT3384 t3384 0 0.1f
M8945 t3382 nw1091 vdd vdd pch w=2u l=180n
M8946 t3382 nw1090 vdd vdd pch w=2u l=180n
CT3385 t3385 0 0.1f
M8947 t3382 nw1091 t3385 0 nch w=1u l=180n
M8948 t3385 nw1090 0 0 nch w=1u l=180n
M8949 t3383 nw1091 vdd vdd pch w=2u l=180n
M8950 t3383 t3382 vdd vdd pch w=2u l=180n
CT3386 t3386 0 0.1f
M8951 t3383 nw1091 t3386 0 nch w=1u l=180n
M8952 t3386 t3382 0 0 nch w=1u l=180n
M8953 t3384 nw1090 vdd vdd pch w=2u l=180n
M8954 t3384 t3382 vdd vdd pch w=2u l=180n
CT3387 t3387 0 0.1f
M8955 t3384 nw1090 t3387 0 nch w=1u l=180n
M8956 t3387 t3382 0 0 nch w=1u l=180n
M8957 nw1092 t3383 vdd vdd pch w=2u l=180n
M8958 nw1092 t3384 vdd vdd pch w=2u l=180n
CT3388 t3388 0 0.1f
M8959 nw1092 t3383 t3388 0 nch w=1u l=180n
M8960 t3388 t3384 0 0 nch w=1u l=180n
Cnw1092 nw1092 0 2f
M8961 nw1093 nw191 vdd vdd pch w=2u l=180n
M8962 nw1093 nw1020 vdd vdd pch w=2u l=180n
CT3389 t3389 0 0.1f
M8963 nw1093 nw191 t3389 0 nch w=1u l=180n
M8964 t3389 nw1020 0 0 nch w=1u l=180n
Cnw1093 nw1093 0 2f
M8965 nw1094 nw1091 vdd vdd pch w=2u l=180n
M8966 nw1094 nw1090 vdd vdd pch w=2u l=180n
CT3390 t3390 0 0.1f
M8967 nw1094 nw1091 t3390 0 nch w=1u l=180n
M8968 t3390 nw1090 0 0 nch w=1u l=180n
Cnw1094 nw1094 0 2f
M8969 nw1095 nw1093 vdd vdd pch w=2u l=180n
M8970 nw1095 nw1094 vdd vdd pch w=2u l=180n
CT3391 t3391 0 0.1f
M8971 nw1095 nw1093 t3391 0 nch w=1u l=180n
M8972 t3391 nw1094 0 0 nch w=1u l=180n
Cnw1095 nw1095 0 2f
CT3392 t3392 0 0.1f
CT3393 t3393 0 0.1f
CT3394 t3394 0 0.1f
M8973 t3392 nw192 vdd vdd pch w=2u l=180n
M8974 t3392 nw1023 vdd vdd pch w=2u l=180n
CT3395 t3395 0 0.1f
M8975 t3392 nw192 t3395 0 nch w=1u l=180n
M8976 t3395 nw1023 0 0 nch w=1u l=180n
M8977 t3393 nw192 vdd vdd pch w=2u l=180n
M8978 t3393 t3392 vdd vdd pch w=2u l=180n
CT3396 t3396 0 0.1f
M8979 t3393 nw192 t3396 0 nch w=1u l=180n
M8980 t3396 t3392 0 0 nch w=1u l=180n
M8981 t3394 nw1023 vdd vdd pch w=2u l=180n
M8982 t3394 t3392 vdd vdd pch w=2u l=180n
CT3397 t3397 0 0.1f
M8983 t3394 nw1023 t3397 0 nch w=1u l=180n
M8984 t3397 t3392 0 0 nch w=1u l=180n
M8985 nw1096 t3393 vdd vdd pch w=2u l=180n
M8986 nw1096 t3394 vdd vdd pch w=2u l=180n
CT3398 t3398 0 0.1f
M8987 nw1096 t3393 t3398 0 nch w=1u l=180n
M8988 t3398 t3394 0 0 nch w=1u l=180n
Cnw1096 nw1096 0 2f
CT3399 t3399 0 0.1f
CT3400 t3400 0 0.1f
CT3401 t3401 0 0.1f
M8989 t3399 nw1096 vdd vdd pch w=2u l=180n
M8990 t3399 nw1095 vdd vdd pch w=2u l=180n
CT3402 t3402 0 0.1f
M8991 t3399 nw1096 t3402 0 nch w=1u l=180n
M8992 t3402 nw1095 0 0 nch w=1u l=180n
M8993 t3400 nw1096 vdd vdd pch w=2u l=180n
M8994 t3400 t3399 vdd vdd pch w=2u l=180n
CT3403 t3403 0 0.1f
M8995 t3400 nw1096 t3403 0 nch w=1u l=180n
M8996 t3403 t3399 0 0 nch w=1u l=180n
M8997 t3401 nw1095 vdd vdd pch w=2u l=180n
M8998 t3401 t3399 vdd vdd pch w=2u l=180n
CT3404 t3404 0 0.1f
M8999 t3401 nw1095 t3404 0 nch w=1u l=180n
M9000 t3404 t3399 0 0 nch w=1u l=180n
M9001 nw1097 t3400 vdd vdd pch w=2u l=180n
M9002 nw1097 t3401 vdd vdd pch w=2u l=180n
CT3405 t3405 0 0.1f
M9003 nw1097 t3400 t3405 0 nch w=1u l=180n
M9004 t3405 t3401 0 0 nch w=1u l=180n
Cnw1097 nw1097 0 2f
M9005 nw1098 nw192 vdd vdd pch w=2u l=180n
M9006 nw1098 nw1023 vdd vdd pch w=2u l=180n
CT3406 t3406 0 0.1f
M9007 nw1098 nw192 t3406 0 nch w=1u l=180n
M9008 t3406 nw1023 0 0 nch w=1u l=180n
Cnw1098 nw1098 0 2f
M9009 nw1099 nw1096 vdd vdd pch w=2u l=180n
M9010 nw1099 nw1095 vdd vdd pch w=2u l=180n
CT3407 t3407 0 0.1f
M9011 nw1099 nw1096 t3407 0 nch w=1u l=180n
M9012 t3407 nw1095 0 0 nch w=1u l=180n
Cnw1099 nw1099 0 2f
M9013 nw1100 nw1098 vdd vdd pch w=2u l=180n
M9014 nw1100 nw1099 vdd vdd pch w=2u l=180n
CT3408 t3408 0 0.1f
M9015 nw1100 nw1098 t3408 0 nch w=1u l=180n
M9016 t3408 nw1099 0 0 nch w=1u l=180n
Cnw1100 nw1100 0 2f
CT3409 t3409 0 0.1f
CT3410 t3410 0 0.1f
CT3411 t3411 0 0.1f
M9017 t3409 nw193 vdd vdd pch w=2u l=180n
M9018 t3409 nw1027 vdd vdd pch w=2u l=180n
CT3412 t3412 0 0.1f
M9019 t3409 nw193 t3412 0 nch w=1u l=180n
M9020 t3412 nw1027 0 0 nch w=1u l=180n
M9021 t3410 nw193 vdd vdd pch w=2u l=180n
M9022 t3410 t3409 vdd vdd pch w=2u l=180n
CT3413 t3413 0 0.1f
M9023 t3410 nw193 t3413 0 nch w=1u l=180n
M9024 t3413 t3409 0 0 nch w=1u l=180n
M9025 t3411 nw1027 vdd vdd pch w=2u l=180n
M9026 t3411 t3409 vdd vdd pch w=2u l=180n
CT3414 t3414 0 0.1f
M9027 t3411 nw1027 t3414 0 nch w=1u l=180n
M9028 t3414 t3409 0 0 nch w=1u l=180n
M9029 nw1101 t3410 vdd vdd pch w=2u l=180n
M9030 nw1101 t3411 vdd vdd pch w=2u l=180n
CT3415 t3415 0 0.1f
M9031 nw1101 t3410 t3415 0 nch w=1u l=180n
M9032 t3415 t3411 0 0 nch w=1u l=180n
Cnw1101 nw1101 0 2f
CT3416 t3416 0 0.1f
M9033 t3416 nw193 vdd vdd pch w=2u l=180n
M9034 t3416 nw1027 vdd vdd pch w=2u l=180n
CT3417 t3417 0 0.1f
M9035 t3416 nw193 t3417 0 nch w=1u l=180n
M9036 t3417 nw1027 0 0 nch w=1u l=180n
M9037 nw1102 t3416 vdd vdd pch w=2u l=180n
M9038 nw1102 t3416 0 0 nch w=1u l=180n
Cnw1102 nw1102 0 2f
CT3418 t3418 0 0.1f
CT3419 t3419 0 0.1f
CT3420 t3420 0 0.1f
M9039 t3418 nw194 vdd vdd pch w=2u l=180n
M9040 t3418 nw1032 vdd vdd pch w=2u l=180n
CT3421 t3421 0 0.1f
M9041 t3418 nw194 t3421 0 nch w=1u l=180n
M9042 t3421 nw1032 0 0 nch w=1u l=180n
M9043 t3419 nw194 vdd vdd pch w=2u l=180n
M9044 t3419 t3418 vdd vdd pch w=2u l=180n
CT3422 t3422 0 0.1f
M9045 t3419 nw194 t3422 0 nch w=1u l=180n
M9046 t3422 t3418 0 0 nch w=1u l=180n
M9047 t3420 nw1032 vdd vdd pch w=2u l=180n
M9048 t3420 t3418 vdd vdd pch w=2u l=180n
CT3423 t3423 0 0.1f
M9049 t3420 nw1032 t3423 0 nch w=1u l=180n
M9050 t3423 t3418 0 0 nch w=1u l=180n
M9051 nw1103 t3419 vdd vdd pch w=2u l=180n
M9052 nw1103 t3420 vdd vdd pch w=2u l=180n
CT3424 t3424 0 0.1f
M9053 nw1103 t3419 t3424 0 nch w=1u l=180n
M9054 t3424 t3420 0 0 nch w=1u l=180n
Cnw1103 nw1103 0 2f
CT3425 t3425 0 0.1f
CT3426 t3426 0 0.1f
CT3427 t3427 0 0.1f
M9055 t3425 nw1103 vdd vdd pch w=2u l=180n
M9056 t3425 nw1102 vdd vdd pch w=2u l=180n
CT3428 t3428 0 0.1f
M9057 t3425 nw1103 t3428 0 nch w=1u l=180n
M9058 t3428 nw1102 0 0 nch w=1u l=180n
M9059 t3426 nw1103 vdd vdd pch w=2u l=180n
M9060 t3426 t3425 vdd vdd pch w=2u l=180n
CT3429 t3429 0 0.1f
M9061 t3426 nw1103 t3429 0 nch w=1u l=180n
M9062 t3429 t3425 0 0 nch w=1u l=180n
M9063 t3427 nw1102 vdd vdd pch w=2u l=180n
M9064 t3427 t3425 vdd vdd pch w=2u l=180n
CT3430 t3430 0 0.1f
M9065 t3427 nw1102 t3430 0 nch w=1u l=180n
M9066 t3430 t3425 0 0 nch w=1u l=180n
M9067 nw1104 t3426 vdd vdd pch w=2u l=180n
M9068 nw1104 t3427 vdd vdd pch w=2u l=180n
CT3431 t3431 0 0.1f
M9069 nw1104 t3426 t3431 0 nch w=1u l=180n
M9070 t3431 t3427 0 0 nch w=1u l=180n
Cnw1104 nw1104 0 2f
M9071 nw1105 nw194 vdd vdd pch w=2u l=180n
M9072 nw1105 nw1032 vdd vdd pch w=2u l=180n
CT3432 t3432 0 0.1f
M9073 nw1105 nw194 t3432 0 nch w=1u l=180n
M9074 t3432 nw1032 0 0 nch w=1u l=180n
Cnw1105 nw1105 0 2f
M9075 nw1106 nw1103 vdd vdd pch w=2u l=180n
M9076 nw1106 nw1102 vdd vdd pch w=2u l=180n
CT3433 t3433 0 0.1f
M9077 nw1106 nw1103 t3433 0 nch w=1u l=180n
M9078 t3433 nw1102 0 0 nch w=1u l=180n
Cnw1106 nw1106 0 2f
M9079 nw1107 nw1105 vdd vdd pch w=2u l=180n
M9080 nw1107 nw1106 vdd vdd pch w=2u l=180n
CT3434 t3434 0 0.1f
M9081 nw1107 nw1105 t3434 0 nch w=1u l=180n
M9082 t3434 nw1106 0 0 nch w=1u l=180n
Cnw1107 nw1107 0 2f
CT3435 t3435 0 0.1f
CT3436 t3436 0 0.1f
CT3437 t3437 0 0.1f
M9083 t3435 nw195 vdd vdd pch w=2u l=180n
M9084 t3435 nw1037 vdd vdd pch w=2u l=180n
CT3438 t3438 0 0.1f
M9085 t3435 nw195 t3438 0 nch w=1u l=180n
M9086 t3438 nw1037 0 0 nch w=1u l=180n
M9087 t3436 nw195 vdd vdd pch w=2u l=180n
M9088 t3436 t3435 vdd vdd pch w=2u l=180n
CT3439 t3439 0 0.1f
M9089 t3436 nw195 t3439 0 nch w=1u l=180n
M9090 t3439 t3435 0 0 nch w=1u l=180n
M9091 t3437 nw1037 vdd vdd pch w=2u l=180n
M9092 t3437 t3435 vdd vdd pch w=2u l=180n
CT3440 t3440 0 0.1f
M9093 t3437 nw1037 t3440 0 nch w=1u l=180n
M9094 t3440 t3435 0 0 nch w=1u l=180n
M9095 nw1108 t3436 vdd vdd pch w=2u l=180n
M9096 nw1108 t3437 vdd vdd pch w=2u l=180n
CT3441 t3441 0 0.1f
M9097 nw1108 t3436 t3441 0 nch w=1u l=180n
M9098 t3441 t3437 0 0 nch w=1u l=180n
Cnw1108 nw1108 0 2f
CT3442 t3442 0 0.1f
CT3443 t3443 0 0.1f
CT3444 t3444 0 0.1f
M9099 t3442 nw1108 vdd vdd pch w=2u l=180n
M9100 t3442 nw1107 vdd vdd pch w=2u l=180n
CT3445 t3445 0 0.1f
M9101 t3442 nw1108 t3445 0 nch w=1u l=180n
M9102 t3445 nw1107 0 0 nch w=1u l=180n
M9103 t3443 nw1108 vdd vdd pch w=2u l=180n
M9104 t3443 t3442 vdd vdd pch w=2u l=180n
CT3446 t3446 0 0.1f
M9105 t3443 nw1108 t3446 0 nch w=1u l=180n
M9106 t3446 t3442 0 0 nch w=1u l=180n
M9107 t3444 nw1107 vdd vdd pch w=2u l=180n
M9108 t3444 t3442 vdd vdd pch w=2u l=180n
CT3447 t3447 0 0.1f
M9109 t3444 nw1107 t3447 0 nch w=1u l=180n
M9110 t3447 t3442 0 0 nch w=1u l=180n
M9111 nw1109 t3443 vdd vdd pch w=2u l=180n
M9112 nw1109 t3444 vdd vdd pch w=2u l=180n
CT3448 t3448 0 0.1f
M9113 nw1109 t3443 t3448 0 nch w=1u l=180n
M9114 t3448 t3444 0 0 nch w=1u l=180n
Cnw1109 nw1109 0 2f
M9115 nw1110 nw195 vdd vdd pch w=2u l=180n
M9116 nw1110 nw1037 vdd vdd pch w=2u l=180n
CT3449 t3449 0 0.1f
M9117 nw1110 nw195 t3449 0 nch w=1u l=180n
M9118 t3449 nw1037 0 0 nch w=1u l=180n
Cnw1110 nw1110 0 2f
M9119 nw1111 nw1108 vdd vdd pch w=2u l=180n
M9120 nw1111 nw1107 vdd vdd pch w=2u l=180n
CT3450 t3450 0 0.1f
M9121 nw1111 nw1108 t3450 0 nch w=1u l=180n
M9122 t3450 nw1107 0 0 nch w=1u l=180n
Cnw1111 nw1111 0 2f
M9123 nw1112 nw1110 vdd vdd pch w=2u l=180n
M9124 nw1112 nw1111 vdd vdd pch w=2u l=180n
CT3451 t3451 0 0.1f
M9125 nw1112 nw1110 t3451 0 nch w=1u l=180n
M9126 t3451 nw1111 0 0 nch w=1u l=180n
Cnw1112 nw1112 0 2f
CT3452 t3452 0 0.1f
CT3453 t3453 0 0.1f
CT3454 t3454 0 0.1f
M9127 t3452 nw196 vdd vdd pch w=2u l=180n
M9128 t3452 nw1042 vdd vdd pch w=2u l=180n
CT3455 t3455 0 0.1f
M9129 t3452 nw196 t3455 0 nch w=1u l=180n
M9130 t3455 nw1042 0 0 nch w=1u l=180n
M9131 t3453 nw196 vdd vdd pch w=2u l=180n
M9132 t3453 t3452 vdd vdd pch w=2u l=180n
CT3456 t3456 0 0.1f
M9133 t3453 nw196 t3456 0 nch w=1u l=180n
M9134 t3456 t3452 0 0 nch w=1u l=180n
M9135 t3454 nw1042 vdd vdd pch w=2u l=180n
M9136 t3454 t3452 vdd vdd pch w=2u l=180n
CT3457 t3457 0 0.1f
M9137 t3454 nw1042 t3457 0 nch w=1u l=180n
M9138 t3457 t3452 0 0 nch w=1u l=180n
M9139 nw1113 t3453 vdd vdd pch w=2u l=180n
M9140 nw1113 t3454 vdd vdd pch w=2u l=180n
CT3458 t3458 0 0.1f
M9141 nw1113 t3453 t3458 0 nch w=1u l=180n
M9142 t3458 t3454 0 0 nch w=1u l=180n
Cnw1113 nw1113 0 2f
CT3459 t3459 0 0.1f
CT3460 t3460 0 0.1f
CT3461 t3461 0 0.1f
M9143 t3459 nw1113 vdd vdd pch w=2u l=180n
M9144 t3459 nw1112 vdd vdd pch w=2u l=180n
CT3462 t3462 0 0.1f
M9145 t3459 nw1113 t3462 0 nch w=1u l=180n
M9146 t3462 nw1112 0 0 nch w=1u l=180n
M9147 t3460 nw1113 vdd vdd pch w=2u l=180n
M9148 t3460 t3459 vdd vdd pch w=2u l=180n
CT3463 t3463 0 0.1f
M9149 t3460 nw1113 t3463 0 nch w=1u l=180n
M9150 t3463 t3459 0 0 nch w=1u l=180n
M9151 t3461 nw1112 vdd vdd pch w=2u l=180n
M9152 t3461 t3459 vdd vdd pch w=2u l=180n
CT3464 t3464 0 0.1f
M9153 t3461 nw1112 t3464 0 nch w=1u l=180n
M9154 t3464 t3459 0 0 nch w=1u l=180n
M9155 nw1114 t3460 vdd vdd pch w=2u l=180n
M9156 nw1114 t3461 vdd vdd pch w=2u l=180n
CT3465 t3465 0 0.1f
M9157 nw1114 t3460 t3465 0 nch w=1u l=180n
M9158 t3465 t3461 0 0 nch w=1u l=180n
Cnw1114 nw1114 0 2f
M9159 nw1115 nw196 vdd vdd pch w=2u l=180n
M9160 nw1115 nw1042 vdd vdd pch w=2u l=180n
CT3466 t3466 0 0.1f
M9161 nw1115 nw196 t3466 0 nch w=1u l=180n
M9162 t3466 nw1042 0 0 nch w=1u l=180n
Cnw1115 nw1115 0 2f
M9163 nw1116 nw1113 vdd vdd pch w=2u l=180n
M9164 nw1116 nw1112 vdd vdd pch w=2u l=180n
CT3467 t3467 0 0.1f
M9165 nw1116 nw1113 t3467 0 nch w=1u l=180n
M9166 t3467 nw1112 0 0 nch w=1u l=180n
Cnw1116 nw1116 0 2f
M9167 nw1117 nw1115 vdd vdd pch w=2u l=180n
M9168 nw1117 nw1116 vdd vdd pch w=2u l=180n
CT3468 t3468 0 0.1f
M9169 nw1117 nw1115 t3468 0 nch w=1u l=180n
M9170 t3468 nw1116 0 0 nch w=1u l=180n
Cnw1117 nw1117 0 2f
CT3469 t3469 0 0.1f
CT3470 t3470 0 0.1f
CT3471 t3471 0 0.1f
M9171 t3469 nw197 vdd vdd pch w=2u l=180n
M9172 t3469 nw1047 vdd vdd pch w=2u l=180n
CT3472 t3472 0 0.1f
M9173 t3469 nw197 t3472 0 nch w=1u l=180n
M9174 t3472 nw1047 0 0 nch w=1u l=180n
M9175 t3470 nw197 vdd vdd pch w=2u l=180n
M9176 t3470 t3469 vdd vdd pch w=2u l=180n
CT3473 t3473 0 0.1f
M9177 t3470 nw197 t3473 0 nch w=1u l=180n
M9178 t3473 t3469 0 0 nch w=1u l=180n
M9179 t3471 nw1047 vdd vdd pch w=2u l=180n
M9180 t3471 t3469 vdd vdd pch w=2u l=180n
CT3474 t3474 0 0.1f
M9181 t3471 nw1047 t3474 0 nch w=1u l=180n
M9182 t3474 t3469 0 0 nch w=1u l=180n
M9183 nw1118 t3470 vdd vdd pch w=2u l=180n
M9184 nw1118 t3471 vdd vdd pch w=2u l=180n
CT3475 t3475 0 0.1f
M9185 nw1118 t3470 t3475 0 nch w=1u l=180n
M9186 t3475 t3471 0 0 nch w=1u l=180n
Cnw1118 nw1118 0 2f
CT3476 t3476 0 0.1f
CT3477 t3477 0 0.1f
CT3478 t3478 0 0.1f
M9187 t3476 nw1118 vdd vdd pch w=2u l=180n
M9188 t3476 nw1117 vdd vdd pch w=2u l=180n
CT3479 t3479 0 0.1f
M9189 t3476 nw1118 t3479 0 nch w=1u l=180n
M9190 t3479 nw1117 0 0 nch w=1u l=180n
M9191 t3477 nw1118 vdd vdd pch w=2u l=180n
M9192 t3477 t3476 vdd vdd pch w=2u l=180n
CT3480 t3480 0 0.1f
M9193 t3477 nw1118 t3480 0 nch w=1u l=180n
M9194 t3480 t3476 0 0 nch w=1u l=180n
M9195 t3478 nw1117 vdd vdd pch w=2u l=180n
M9196 t3478 t3476 vdd vdd pch w=2u l=180n
CT3481 t3481 0 0.1f
M9197 t3478 nw1117 t3481 0 nch w=1u l=180n
M9198 t3481 t3476 0 0 nch w=1u l=180n
M9199 nw1119 t3477 vdd vdd pch w=2u l=180n
M9200 nw1119 t3478 vdd vdd pch w=2u l=180n
CT3482 t3482 0 0.1f
M9201 nw1119 t3477 t3482 0 nch w=1u l=180n
M9202 t3482 t3478 0 0 nch w=1u l=180n
Cnw1119 nw1119 0 2f
M9203 nw1120 nw197 vdd vdd pch w=2u l=180n
M9204 nw1120 nw1047 vdd vdd pch w=2u l=180n
CT3483 t3483 0 0.1f
M9205 nw1120 nw197 t3483 0 nch w=1u l=180n
M9206 t3483 nw1047 0 0 nch w=1u l=180n
Cnw1120 nw1120 0 2f
M9207 nw1121 nw1118 vdd vdd pch w=2u l=180n
M9208 nw1121 nw1117 vdd vdd pch w=2u l=180n
CT3484 t3484 0 0.1f
M9209 nw1121 nw1118 t3484 0 nch w=1u l=180n
M9210 t3484 nw1117 0 0 nch w=1u l=180n
Cnw1121 nw1121 0 2f
M9211 nw1122 nw1120 vdd vdd pch w=2u l=180n
M9212 nw1122 nw1121 vdd vdd pch w=2u l=180n
CT3485 t3485 0 0.1f
M9213 nw1122 nw1120 t3485 0 nch w=1u l=180n
M9214 t3485 nw1121 0 0 nch w=1u l=180n
Cnw1122 nw1122 0 2f
CT3486 t3486 0 0.1f
CT3487 t3487 0 0.1f
CT3488 t3488 0 0.1f
M9215 t3486 nw198 vdd vdd pch w=2u l=180n
M9216 t3486 nw1052 vdd vdd pch w=2u l=180n
CT3489 t3489 0 0.1f
M9217 t3486 nw198 t3489 0 nch w=1u l=180n
M9218 t3489 nw1052 0 0 nch w=1u l=180n
M9219 t3487 nw198 vdd vdd pch w=2u l=180n
M9220 t3487 t3486 vdd vdd pch w=2u l=180n
CT3490 t3490 0 0.1f
M9221 t3487 nw198 t3490 0 nch w=1u l=180n
M9222 t3490 t3486 0 0 nch w=1u l=180n
M9223 t3488 nw1052 vdd vdd pch w=2u l=180n
M9224 t3488 t3486 vdd vdd pch w=2u l=180n
CT3491 t3491 0 0.1f
M9225 t3488 nw1052 t3491 0 nch w=1u l=180n
M9226 t3491 t3486 0 0 nch w=1u l=180n
M9227 nw1123 t3487 vdd vdd pch w=2u l=180n
M9228 nw1123 t3488 vdd vdd pch w=2u l=180n
CT3492 t3492 0 0.1f
M9229 nw1123 t3487 t3492 0 nch w=1u l=180n
M9230 t3492 t3488 0 0 nch w=1u l=180n
Cnw1123 nw1123 0 2f
CT3493 t3493 0 0.1f
CT3494 t3494 0 0.1f
CT3495 t3495 0 0.1f
M9231 t3493 nw1123 vdd vdd pch w=2u l=180n
M9232 t3493 nw1122 vdd vdd pch w=2u l=180n
CT3496 t3496 0 0.1f
M9233 t3493 nw1123 t3496 0 nch w=1u l=180n
M9234 t3496 nw1122 0 0 nch w=1u l=180n
M9235 t3494 nw1123 vdd vdd pch w=2u l=180n
M9236 t3494 t3493 vdd vdd pch w=2u l=180n
CT3497 t3497 0 0.1f
M9237 t3494 nw1123 t3497 0 nch w=1u l=180n
M9238 t3497 t3493 0 0 nch w=1u l=180n
M9239 t3495 nw1122 vdd vdd pch w=2u l=180n
M9240 t3495 t3493 vdd vdd pch w=2u l=180n
CT3498 t3498 0 0.1f
M9241 t3495 nw1122 t3498 0 nch w=1u l=180n
M9242 t3498 t3493 0 0 nch w=1u l=180n
M9243 nw1124 t3494 vdd vdd pch w=2u l=180n
M9244 nw1124 t3495 vdd vdd pch w=2u l=180n
CT3499 t3499 0 0.1f
M9245 nw1124 t3494 t3499 0 nch w=1u l=180n
M9246 t3499 t3495 0 0 nch w=1u l=180n
Cnw1124 nw1124 0 2f
M9247 nw1125 nw198 vdd vdd pch w=2u l=180n
M9248 nw1125 nw1052 vdd vdd pch w=2u l=180n
CT3500 t3500 0 0.1f
M9249 nw1125 nw198 t3500 0 nch w=1u l=180n
M9250 t3500 nw1052 0 0 nch w=1u l=180n
Cnw1125 nw1125 0 2f
M9251 nw1126 nw1123 vdd vdd pch w=2u l=180n
M9252 nw1126 nw1122 vdd vdd pch w=2u l=180n
CT3501 t3501 0 0.1f
M9253 nw1126 nw1123 t3501 0 nch w=1u l=180n
M9254 t3501 nw1122 0 0 nch w=1u l=180n
Cnw1126 nw1126 0 2f
M9255 nw1127 nw1125 vdd vdd pch w=2u l=180n
M9256 nw1127 nw1126 vdd vdd pch w=2u l=180n
CT3502 t3502 0 0.1f
M9257 nw1127 nw1125 t3502 0 nch w=1u l=180n
M9258 t3502 nw1126 0 0 nch w=1u l=180n
Cnw1127 nw1127 0 2f
CT3503 t3503 0 0.1f
CT3504 t3504 0 0.1f
CT3505 t3505 0 0.1f
M9259 t3503 nw199 vdd vdd pch w=2u l=180n
M9260 t3503 nw1057 vdd vdd pch w=2u l=180n
CT3506 t3506 0 0.1f
M9261 t3503 nw199 t3506 0 nch w=1u l=180n
M9262 t3506 nw1057 0 0 nch w=1u l=180n
M9263 t3504 nw199 vdd vdd pch w=2u l=180n
M9264 t3504 t3503 vdd vdd pch w=2u l=180n
CT3507 t3507 0 0.1f
M9265 t3504 nw199 t3507 0 nch w=1u l=180n
M9266 t3507 t3503 0 0 nch w=1u l=180n
M9267 t3505 nw1057 vdd vdd pch w=2u l=180n
M9268 t3505 t3503 vdd vdd pch w=2u l=180n
CT3508 t3508 0 0.1f
M9269 t3505 nw1057 t3508 0 nch w=1u l=180n
M9270 t3508 t3503 0 0 nch w=1u l=180n
M9271 nw1128 t3504 vdd vdd pch w=2u l=180n
M9272 nw1128 t3505 vdd vdd pch w=2u l=180n
CT3509 t3509 0 0.1f
M9273 nw1128 t3504 t3509 0 nch w=1u l=180n
M9274 t3509 t3505 0 0 nch w=1u l=180n
Cnw1128 nw1128 0 2f
CT3510 t3510 0 0.1f
CT3511 t3511 0 0.1f
CT3512 t3512 0 0.1f
M9275 t3510 nw1128 vdd vdd pch w=2u l=180n
M9276 t3510 nw1127 vdd vdd pch w=2u l=180n
CT3513 t3513 0 0.1f
M9277 t3510 nw1128 t3513 0 nch w=1u l=180n
M9278 t3513 nw1127 0 0 nch w=1u l=180n
M9279 t3511 nw1128 vdd vdd pch w=2u l=180n
M9280 t3511 t3510 vdd vdd pch w=2u l=180n
CT3514 t3514 0 0.1f
M9281 t3511 nw1128 t3514 0 nch w=1u l=180n
M9282 t3514 t3510 0 0 nch w=1u l=180n
M9283 t3512 nw1127 vdd vdd pch w=2u l=180n
M9284 t3512 t3510 vdd vdd pch w=2u l=180n
CT3515 t3515 0 0.1f
M9285 t3512 nw1127 t3515 0 nch w=1u l=180n
M9286 t3515 t3510 0 0 nch w=1u l=180n
M9287 nw1129 t3511 vdd vdd pch w=2u l=180n
M9288 nw1129 t3512 vdd vdd pch w=2u l=180n
CT3516 t3516 0 0.1f
M9289 nw1129 t3511 t3516 0 nch w=1u l=180n
M9290 t3516 t3512 0 0 nch w=1u l=180n
Cnw1129 nw1129 0 2f
M9291 nw1130 nw199 vdd vdd pch w=2u l=180n
M9292 nw1130 nw1057 vdd vdd pch w=2u l=180n
CT3517 t3517 0 0.1f
M9293 nw1130 nw199 t3517 0 nch w=1u l=180n
M9294 t3517 nw1057 0 0 nch w=1u l=180n
Cnw1130 nw1130 0 2f
M9295 nw1131 nw1128 vdd vdd pch w=2u l=180n
M9296 nw1131 nw1127 vdd vdd pch w=2u l=180n
CT3518 t3518 0 0.1f
M9297 nw1131 nw1128 t3518 0 nch w=1u l=180n
M9298 t3518 nw1127 0 0 nch w=1u l=180n
Cnw1131 nw1131 0 2f
M9299 nw1132 nw1130 vdd vdd pch w=2u l=180n
M9300 nw1132 nw1131 vdd vdd pch w=2u l=180n
CT3519 t3519 0 0.1f
M9301 nw1132 nw1130 t3519 0 nch w=1u l=180n
M9302 t3519 nw1131 0 0 nch w=1u l=180n
Cnw1132 nw1132 0 2f
CT3520 t3520 0 0.1f
CT3521 t3521 0 0.1f
CT3522 t3522 0 0.1f
M9303 t3520 nw200 vdd vdd pch w=2u l=180n
M9304 t3520 nw1062 vdd vdd pch w=2u l=180n
CT3523 t3523 0 0.1f
M9305 t3520 nw200 t3523 0 nch w=1u l=180n
M9306 t3523 nw1062 0 0 nch w=1u l=180n
M9307 t3521 nw200 vdd vdd pch w=2u l=180n
M9308 t3521 t3520 vdd vdd pch w=2u l=180n
CT3524 t3524 0 0.1f
M9309 t3521 nw200 t3524 0 nch w=1u l=180n
M9310 t3524 t3520 0 0 nch w=1u l=180n
M9311 t3522 nw1062 vdd vdd pch w=2u l=180n
M9312 t3522 t3520 vdd vdd pch w=2u l=180n
CT3525 t3525 0 0.1f
M9313 t3522 nw1062 t3525 0 nch w=1u l=180n
M9314 t3525 t3520 0 0 nch w=1u l=180n
M9315 nw1133 t3521 vdd vdd pch w=2u l=180n
M9316 nw1133 t3522 vdd vdd pch w=2u l=180n
CT3526 t3526 0 0.1f
M9317 nw1133 t3521 t3526 0 nch w=1u l=180n
M9318 t3526 t3522 0 0 nch w=1u l=180n
Cnw1133 nw1133 0 2f
CT3527 t3527 0 0.1f
CT3528 t3528 0 0.1f
CT3529 t3529 0 0.1f
M9319 t3527 nw1133 vdd vdd pch w=2u l=180n
M9320 t3527 nw1132 vdd vdd pch w=2u l=180n
CT3530 t3530 0 0.1f
M9321 t3527 nw1133 t3530 0 nch w=1u l=180n
M9322 t3530 nw1132 0 0 nch w=1u l=180n
M9323 t3528 nw1133 vdd vdd pch w=2u l=180n
M9324 t3528 t3527 vdd vdd pch w=2u l=180n
CT3531 t3531 0 0.1f
M9325 t3528 nw1133 t3531 0 nch w=1u l=180n
M9326 t3531 t3527 0 0 nch w=1u l=180n
M9327 t3529 nw1132 vdd vdd pch w=2u l=180n
M9328 t3529 t3527 vdd vdd pch w=2u l=180n
CT3532 t3532 0 0.1f
M9329 t3529 nw1132 t3532 0 nch w=1u l=180n
M9330 t3532 t3527 0 0 nch w=1u l=180n
M9331 nw1134 t3528 vdd vdd pch w=2u l=180n
M9332 nw1134 t3529 vdd vdd pch w=2u l=180n
CT3533 t3533 0 0.1f
M9333 nw1134 t3528 t3533 0 nch w=1u l=180n
M9334 t3533 t3529 0 0 nch w=1u l=180n
Cnw1134 nw1134 0 2f
M9335 nw1135 nw200 vdd vdd pch w=2u l=180n
M9336 nw1135 nw1062 vdd vdd pch w=2u l=180n
CT3534 t3534 0 0.1f
M9337 nw1135 nw200 t3534 0 nch w=1u l=180n
M9338 t3534 nw1062 0 0 nch w=1u l=180n
Cnw1135 nw1135 0 2f
M9339 nw1136 nw1133 vdd vdd pch w=2u l=180n
M9340 nw1136 nw1132 vdd vdd pch w=2u l=180n
CT3535 t3535 0 0.1f
M9341 nw1136 nw1133 t3535 0 nch w=1u l=180n
M9342 t3535 nw1132 0 0 nch w=1u l=180n
Cnw1136 nw1136 0 2f
M9343 nw1137 nw1135 vdd vdd pch w=2u l=180n
M9344 nw1137 nw1136 vdd vdd pch w=2u l=180n
CT3536 t3536 0 0.1f
M9345 nw1137 nw1135 t3536 0 nch w=1u l=180n
M9346 t3536 nw1136 0 0 nch w=1u l=180n
Cnw1137 nw1137 0 2f
CT3537 t3537 0 0.1f
CT3538 t3538 0 0.1f
CT3539 t3539 0 0.1f
M9347 t3537 nw201 vdd vdd pch w=2u l=180n
M9348 t3537 nw1067 vdd vdd pch w=2u l=180n
CT3540 t3540 0 0.1f
M9349 t3537 nw201 t3540 0 nch w=1u l=180n
M9350 t3540 nw1067 0 0 nch w=1u l=180n
M9351 t3538 nw201 vdd vdd pch w=2u l=180n
M9352 t3538 t3537 vdd vdd pch w=2u l=180n
CT3541 t3541 0 0.1f
M9353 t3538 nw201 t3541 0 nch w=1u l=180n
M9354 t3541 t3537 0 0 nch w=1u l=180n
M9355 t3539 nw1067 vdd vdd pch w=2u l=180n
M9356 t3539 t3537 vdd vdd pch w=2u l=180n
CT3542 t3542 0 0.1f
M9357 t3539 nw1067 t3542 0 nch w=1u l=180n
M9358 t3542 t3537 0 0 nch w=1u l=180n
M9359 nw1138 t3538 vdd vdd pch w=2u l=180n
M9360 nw1138 t3539 vdd vdd pch w=2u l=180n
CT3543 t3543 0 0.1f
M9361 nw1138 t3538 t3543 0 nch w=1u l=180n
M9362 t3543 t3539 0 0 nch w=1u l=180n
Cnw1138 nw1138 0 2f
CT3544 t3544 0 0.1f
CT3545 t3545 0 0.1f
CT3546 t3546 0 0.1f
M9363 t3544 nw1138 vdd vdd pch w=2u l=180n
M9364 t3544 nw1137 vdd vdd pch w=2u l=180n
CT3547 t3547 0 0.1f
M9365 t3544 nw1138 t3547 0 nch w=1u l=180n
M9366 t3547 nw1137 0 0 nch w=1u l=180n
M9367 t3545 nw1138 vdd vdd pch w=2u l=180n
M9368 t3545 t3544 vdd vdd pch w=2u l=180n
CT3548 t3548 0 0.1f
M9369 t3545 nw1138 t3548 0 nch w=1u l=180n
M9370 t3548 t3544 0 0 nch w=1u l=180n
M9371 t3546 nw1137 vdd vdd pch w=2u l=180n
M9372 t3546 t3544 vdd vdd pch w=2u l=180n
CT3549 t3549 0 0.1f
M9373 t3546 nw1137 t3549 0 nch w=1u l=180n
M9374 t3549 t3544 0 0 nch w=1u l=180n
M9375 nw1139 t3545 vdd vdd pch w=2u l=180n
M9376 nw1139 t3546 vdd vdd pch w=2u l=180n
CT3550 t3550 0 0.1f
M9377 nw1139 t3545 t3550 0 nch w=1u l=180n
M9378 t3550 t3546 0 0 nch w=1u l=180n
Cnw1139 nw1139 0 2f
M9379 nw1140 nw201 vdd vdd pch w=2u l=180n
M9380 nw1140 nw1067 vdd vdd pch w=2u l=180n
CT3551 t3551 0 0.1f
M9381 nw1140 nw201 t3551 0 nch w=1u l=180n
M9382 t3551 nw1067 0 0 nch w=1u l=180n
Cnw1140 nw1140 0 2f
M9383 nw1141 nw1138 vdd vdd pch w=2u l=180n
M9384 nw1141 nw1137 vdd vdd pch w=2u l=180n
CT3552 t3552 0 0.1f
M9385 nw1141 nw1138 t3552 0 nch w=1u l=180n
M9386 t3552 nw1137 0 0 nch w=1u l=180n
Cnw1141 nw1141 0 2f
M9387 nw1142 nw1140 vdd vdd pch w=2u l=180n
M9388 nw1142 nw1141 vdd vdd pch w=2u l=180n
CT3553 t3553 0 0.1f
M9389 nw1142 nw1140 t3553 0 nch w=1u l=180n
M9390 t3553 nw1141 0 0 nch w=1u l=180n
Cnw1142 nw1142 0 2f
CT3554 t3554 0 0.1f
CT3555 t3555 0 0.1f
CT3556 t3556 0 0.1f
M9391 t3554 nw202 vdd vdd pch w=2u l=180n
M9392 t3554 nw1072 vdd vdd pch w=2u l=180n
CT3557 t3557 0 0.1f
M9393 t3554 nw202 t3557 0 nch w=1u l=180n
M9394 t3557 nw1072 0 0 nch w=1u l=180n
M9395 t3555 nw202 vdd vdd pch w=2u l=180n
M9396 t3555 t3554 vdd vdd pch w=2u l=180n
CT3558 t3558 0 0.1f
M9397 t3555 nw202 t3558 0 nch w=1u l=180n
M9398 t3558 t3554 0 0 nch w=1u l=180n
M9399 t3556 nw1072 vdd vdd pch w=2u l=180n
M9400 t3556 t3554 vdd vdd pch w=2u l=180n
CT3559 t3559 0 0.1f
M9401 t3556 nw1072 t3559 0 nch w=1u l=180n
M9402 t3559 t3554 0 0 nch w=1u l=180n
M9403 nw1143 t3555 vdd vdd pch w=2u l=180n
M9404 nw1143 t3556 vdd vdd pch w=2u l=180n
CT3560 t3560 0 0.1f
M9405 nw1143 t3555 t3560 0 nch w=1u l=180n
M9406 t3560 t3556 0 0 nch w=1u l=180n
Cnw1143 nw1143 0 2f
CT3561 t3561 0 0.1f
CT3562 t3562 0 0.1f
CT3563 t3563 0 0.1f
M9407 t3561 nw1143 vdd vdd pch w=2u l=180n
M9408 t3561 nw1142 vdd vdd pch w=2u l=180n
CT3564 t3564 0 0.1f
M9409 t3561 nw1143 t3564 0 nch w=1u l=180n
M9410 t3564 nw1142 0 0 nch w=1u l=180n
M9411 t3562 nw1143 vdd vdd pch w=2u l=180n
M9412 t3562 t3561 vdd vdd pch w=2u l=180n
CT3565 t3565 0 0.1f
M9413 t3562 nw1143 t3565 0 nch w=1u l=180n
M9414 t3565 t3561 0 0 nch w=1u l=180n
M9415 t3563 nw1142 vdd vdd pch w=2u l=180n
M9416 t3563 t3561 vdd vdd pch w=2u l=180n
CT3566 t3566 0 0.1f
M9417 t3563 nw1142 t3566 0 nch w=1u l=180n
M9418 t3566 t3561 0 0 nch w=1u l=180n
M9419 nw1144 t3562 vdd vdd pch w=2u l=180n
M9420 nw1144 t3563 vdd vdd pch w=2u l=180n
CT3567 t3567 0 0.1f
M9421 nw1144 t3562 t3567 0 nch w=1u l=180n
M9422 t3567 t3563 0 0 nch w=1u l=180n
Cnw1144 nw1144 0 2f
M9423 nw1145 nw202 vdd vdd pch w=2u l=180n
M9424 nw1145 nw1072 vdd vdd pch w=2u l=180n
CT3568 t3568 0 0.1f
M9425 nw1145 nw202 t3568 0 nch w=1u l=180n
M9426 t3568 nw1072 0 0 nch w=1u l=180n
Cnw1145 nw1145 0 2f
M9427 nw1146 nw1143 vdd vdd pch w=2u l=180n
M9428 nw1146 nw1142 vdd vdd pch w=2u l=180n
CT3569 t3569 0 0.1f
M9429 nw1146 nw1143 t3569 0 nch w=1u l=180n
M9430 t3569 nw1142 0 0 nch w=1u l=180n
Cnw1146 nw1146 0 2f
M9431 nw1147 nw1145 vdd vdd pch w=2u l=180n
M9432 nw1147 nw1146 vdd vdd pch w=2u l=180n
CT3570 t3570 0 0.1f
M9433 nw1147 nw1145 t3570 0 nch w=1u l=180n
M9434 t3570 nw1146 0 0 nch w=1u l=180n
Cnw1147 nw1147 0 2f
CT3571 t3571 0 0.1f
CT3572 t3572 0 0.1f
CT3573 t3573 0 0.1f
M9435 t3571 nw203 vdd vdd pch w=2u l=180n
M9436 t3571 nw1077 vdd vdd pch w=2u l=180n
CT3574 t3574 0 0.1f
M9437 t3571 nw203 t3574 0 nch w=1u l=180n
M9438 t3574 nw1077 0 0 nch w=1u l=180n
M9439 t3572 nw203 vdd vdd pch w=2u l=180n
M9440 t3572 t3571 vdd vdd pch w=2u l=180n
CT3575 t3575 0 0.1f
M9441 t3572 nw203 t3575 0 nch w=1u l=180n
M9442 t3575 t3571 0 0 nch w=1u l=180n
M9443 t3573 nw1077 vdd vdd pch w=2u l=180n
M9444 t3573 t3571 vdd vdd pch w=2u l=180n
CT3576 t3576 0 0.1f
M9445 t3573 nw1077 t3576 0 nch w=1u l=180n
M9446 t3576 t3571 0 0 nch w=1u l=180n
M9447 nw1148 t3572 vdd vdd pch w=2u l=180n
M9448 nw1148 t3573 vdd vdd pch w=2u l=180n
CT3577 t3577 0 0.1f
M9449 nw1148 t3572 t3577 0 nch w=1u l=180n
M9450 t3577 t3573 0 0 nch w=1u l=180n
Cnw1148 nw1148 0 2f
CT3578 t3578 0 0.1f
CT3579 t3579 0 0.1f
CT3580 t3580 0 0.1f
M9451 t3578 nw1148 vdd vdd pch w=2u l=180n
M9452 t3578 nw1147 vdd vdd pch w=2u l=180n
CT3581 t3581 0 0.1f
M9453 t3578 nw1148 t3581 0 nch w=1u l=180n
M9454 t3581 nw1147 0 0 nch w=1u l=180n
M9455 t3579 nw1148 vdd vdd pch w=2u l=180n
M9456 t3579 t3578 vdd vdd pch w=2u l=180n
CT3582 t3582 0 0.1f
M9457 t3579 nw1148 t3582 0 nch w=1u l=180n
M9458 t3582 t3578 0 0 nch w=1u l=180n
M9459 t3580 nw1147 vdd vdd pch w=2u l=180n
M9460 t3580 t3578 vdd vdd pch w=2u l=180n
CT3583 t3583 0 0.1f
M9461 t3580 nw1147 t3583 0 nch w=1u l=180n
M9462 t3583 t3578 0 0 nch w=1u l=180n
M9463 nw1149 t3579 vdd vdd pch w=2u l=180n
M9464 nw1149 t3580 vdd vdd pch w=2u l=180n
CT3584 t3584 0 0.1f
M9465 nw1149 t3579 t3584 0 nch w=1u l=180n
M9466 t3584 t3580 0 0 nch w=1u l=180n
Cnw1149 nw1149 0 2f
M9467 nw1150 nw203 vdd vdd pch w=2u l=180n
M9468 nw1150 nw1077 vdd vdd pch w=2u l=180n
CT3585 t3585 0 0.1f
M9469 nw1150 nw203 t3585 0 nch w=1u l=180n
M9470 t3585 nw1077 0 0 nch w=1u l=180n
Cnw1150 nw1150 0 2f
M9471 nw1151 nw1148 vdd vdd pch w=2u l=180n
M9472 nw1151 nw1147 vdd vdd pch w=2u l=180n
CT3586 t3586 0 0.1f
M9473 nw1151 nw1148 t3586 0 nch w=1u l=180n
M9474 t3586 nw1147 0 0 nch w=1u l=180n
Cnw1151 nw1151 0 2f
M9475 nw1152 nw1150 vdd vdd pch w=2u l=180n
M9476 nw1152 nw1151 vdd vdd pch w=2u l=180n
CT3587 t3587 0 0.1f
M9477 nw1152 nw1150 t3587 0 nch w=1u l=180n
M9478 t3587 nw1151 0 0 nch w=1u l=180n
Cnw1152 nw1152 0 2f
CT3588 t3588 0 0.1f
CT3589 t3589 0 0.1f
CT3590 t3590 0 0.1f
M9479 t3588 nw204 vdd vdd pch w=2u l=180n
M9480 t3588 nw1082 vdd vdd pch w=2u l=180n
CT3591 t3591 0 0.1f
M9481 t3588 nw204 t3591 0 nch w=1u l=180n
M9482 t3591 nw1082 0 0 nch w=1u l=180n
M9483 t3589 nw204 vdd vdd pch w=2u l=180n
M9484 t3589 t3588 vdd vdd pch w=2u l=180n
CT3592 t3592 0 0.1f
M9485 t3589 nw204 t3592 0 nch w=1u l=180n
M9486 t3592 t3588 0 0 nch w=1u l=180n
M9487 t3590 nw1082 vdd vdd pch w=2u l=180n
M9488 t3590 t3588 vdd vdd pch w=2u l=180n
CT3593 t3593 0 0.1f
M9489 t3590 nw1082 t3593 0 nch w=1u l=180n
M9490 t3593 t3588 0 0 nch w=1u l=180n
M9491 nw1153 t3589 vdd vdd pch w=2u l=180n
M9492 nw1153 t3590 vdd vdd pch w=2u l=180n
CT3594 t3594 0 0.1f
M9493 nw1153 t3589 t3594 0 nch w=1u l=180n
M9494 t3594 t3590 0 0 nch w=1u l=180n
Cnw1153 nw1153 0 2f
CT3595 t3595 0 0.1f
CT3596 t3596 0 0.1f
CT3597 t3597 0 0.1f
M9495 t3595 nw1153 vdd vdd pch w=2u l=180n
M9496 t3595 nw1152 vdd vdd pch w=2u l=180n
CT3598 t3598 0 0.1f
M9497 t3595 nw1153 t3598 0 nch w=1u l=180n
M9498 t3598 nw1152 0 0 nch w=1u l=180n
M9499 t3596 nw1153 vdd vdd pch w=2u l=180n
M9500 t3596 t3595 vdd vdd pch w=2u l=180n
CT3599 t3599 0 0.1f
M9501 t3596 nw1153 t3599 0 nch w=1u l=180n
M9502 t3599 t3595 0 0 nch w=1u l=180n
M9503 t3597 nw1152 vdd vdd pch w=2u l=180n
M9504 t3597 t3595 vdd vdd pch w=2u l=180n
CT3600 t3600 0 0.1f
M9505 t3597 nw1152 t3600 0 nch w=1u l=180n
M9506 t3600 t3595 0 0 nch w=1u l=180n
M9507 nw1154 t3596 vdd vdd pch w=2u l=180n
M9508 nw1154 t3597 vdd vdd pch w=2u l=180n
CT3601 t3601 0 0.1f
M9509 nw1154 t3596 t3601 0 nch w=1u l=180n
M9510 t3601 t3597 0 0 nch w=1u l=180n
Cnw1154 nw1154 0 2f
M9511 nw1155 nw204 vdd vdd pch w=2u l=180n
M9512 nw1155 nw1082 vdd vdd pch w=2u l=180n
CT3602 t3602 0 0.1f
M9513 nw1155 nw204 t3602 0 nch w=1u l=180n
M9514 t3602 nw1082 0 0 nch w=1u l=180n
Cnw1155 nw1155 0 2f
M9515 nw1156 nw1153 vdd vdd pch w=2u l=180n
M9516 nw1156 nw1152 vdd vdd pch w=2u l=180n
CT3603 t3603 0 0.1f
M9517 nw1156 nw1153 t3603 0 nch w=1u l=180n
M9518 t3603 nw1152 0 0 nch w=1u l=180n
Cnw1156 nw1156 0 2f
M9519 nw1157 nw1155 vdd vdd pch w=2u l=180n
M9520 nw1157 nw1156 vdd vdd pch w=2u l=180n
CT3604 t3604 0 0.1f
M9521 nw1157 nw1155 t3604 0 nch w=1u l=180n
M9522 t3604 nw1156 0 0 nch w=1u l=180n
Cnw1157 nw1157 0 2f
CT3605 t3605 0 0.1f
CT3606 t3606 0 0.1f
CT3607 t3607 0 0.1f
M9523 t3605 nw205 vdd vdd pch w=2u l=180n
M9524 t3605 nw1087 vdd vdd pch w=2u l=180n
CT3608 t3608 0 0.1f
M9525 t3605 nw205 t3608 0 nch w=1u l=180n
M9526 t3608 nw1087 0 0 nch w=1u l=180n
M9527 t3606 nw205 vdd vdd pch w=2u l=180n
M9528 t3606 t3605 vdd vdd pch w=2u l=180n
CT3609 t3609 0 0.1f
M9529 t3606 nw205 t3609 0 nch w=1u l=180n
M9530 t3609 t3605 0 0 nch w=1u l=180n
M9531 t3607 nw1087 vdd vdd pch w=2u l=180n
M9532 t3607 t3605 vdd vdd pch w=2u l=180n
CT3610 t3610 0 0.1f
M9533 t3607 nw1087 t3610 0 nch w=1u l=180n
M9534 t3610 t3605 0 0 nch w=1u l=180n
M9535 nw1158 t3606 vdd vdd pch w=2u l=180n
M9536 nw1158 t3607 vdd vdd pch w=2u l=180n
CT3611 t3611 0 0.1f
M9537 nw1158 t3606 t3611 0 nch w=1u l=180n
M9538 t3611 t3607 0 0 nch w=1u l=180n
Cnw1158 nw1158 0 2f
CT3612 t3612 0 0.1f
CT3613 t3613 0 0.1f
CT3614 t3614 0 0.1f
M9539 t3612 nw1158 vdd vdd pch w=2u l=180n
M9540 t3612 nw1157 vdd vdd pch w=2u l=180n
CT3615 t3615 0 0.1f
M9541 t3612 nw1158 t3615 0 nch w=1u l=180n
M9542 t3615 nw1157 0 0 nch w=1u l=180n
M9543 t3613 nw1158 vdd vdd pch w=2u l=180n
M9544 t3613 t3612 vdd vdd pch w=2u l=180n
CT3616 t3616 0 0.1f
M9545 t3613 nw1158 t3616 0 nch w=1u l=180n
M9546 t3616 t3612 0 0 nch w=1u l=180n
M9547 t3614 nw1157 vdd vdd pch w=2u l=180n
M9548 t3614 t3612 vdd vdd pch w=2u l=180n
CT3617 t3617 0 0.1f
M9549 t3614 nw1157 t3617 0 nch w=1u l=180n
M9550 t3617 t3612 0 0 nch w=1u l=180n
M9551 nw1159 t3613 vdd vdd pch w=2u l=180n
M9552 nw1159 t3614 vdd vdd pch w=2u l=180n
CT3618 t3618 0 0.1f
M9553 nw1159 t3613 t3618 0 nch w=1u l=180n
M9554 t3618 t3614 0 0 nch w=1u l=180n
Cnw1159 nw1159 0 2f
M9555 nw1160 nw205 vdd vdd pch w=2u l=180n
M9556 nw1160 nw1087 vdd vdd pch w=2u l=180n
CT3619 t3619 0 0.1f
M9557 nw1160 nw205 t3619 0 nch w=1u l=180n
M9558 t3619 nw1087 0 0 nch w=1u l=180n
Cnw1160 nw1160 0 2f
M9559 nw1161 nw1158 vdd vdd pch w=2u l=180n
M9560 nw1161 nw1157 vdd vdd pch w=2u l=180n
CT3620 t3620 0 0.1f
M9561 nw1161 nw1158 t3620 0 nch w=1u l=180n
M9562 t3620 nw1157 0 0 nch w=1u l=180n
Cnw1161 nw1161 0 2f
M9563 nw1162 nw1160 vdd vdd pch w=2u l=180n
M9564 nw1162 nw1161 vdd vdd pch w=2u l=180n
CT3621 t3621 0 0.1f
M9565 nw1162 nw1160 t3621 0 nch w=1u l=180n
M9566 t3621 nw1161 0 0 nch w=1u l=180n
Cnw1162 nw1162 0 2f
CT3622 t3622 0 0.1f
CT3623 t3623 0 0.1f
CT3624 t3624 0 0.1f
M9567 t3622 nw206 vdd vdd pch w=2u l=180n
M9568 t3622 nw1092 vdd vdd pch w=2u l=180n
CT3625 t3625 0 0.1f
M9569 t3622 nw206 t3625 0 nch w=1u l=180n
M9570 t3625 nw1092 0 0 nch w=1u l=180n
M9571 t3623 nw206 vdd vdd pch w=2u l=180n
M9572 t3623 t3622 vdd vdd pch w=2u l=180n
CT3626 t3626 0 0.1f
M9573 t3623 nw206 t3626 0 nch w=1u l=180n
M9574 t3626 t3622 0 0 nch w=1u l=180n
M9575 t3624 nw1092 vdd vdd pch w=2u l=180n
M9576 t3624 t3622 vdd vdd pch w=2u l=180n
CT3627 t3627 0 0.1f
M9577 t3624 nw1092 t3627 0 nch w=1u l=180n
M9578 t3627 t3622 0 0 nch w=1u l=180n
M9579 nw1163 t3623 vdd vdd pch w=2u l=180n
M9580 nw1163 t3624 vdd vdd pch w=2u l=180n
CT3628 t3628 0 0.1f
M9581 nw1163 t3623 t3628 0 nch w=1u l=180n
M9582 t3628 t3624 0 0 nch w=1u l=180n
Cnw1163 nw1163 0 2f
CT3629 t3629 0 0.1f
CT3630 t3630 0 0.1f
CT3631 t3631 0 0.1f
M9583 t3629 nw1163 vdd vdd pch w=2u l=180n
M9584 t3629 nw1162 vdd vdd pch w=2u l=180n
CT3632 t3632 0 0.1f
M9585 t3629 nw1163 t3632 0 nch w=1u l=180n
M9586 t3632 nw1162 0 0 nch w=1u l=180n
M9587 t3630 nw1163 vdd vdd pch w=2u l=180n
M9588 t3630 t3629 vdd vdd pch w=2u l=180n
CT3633 t3633 0 0.1f
M9589 t3630 nw1163 t3633 0 nch w=1u l=180n
M9590 t3633 t3629 0 0 nch w=1u l=180n
M9591 t3631 nw1162 vdd vdd pch w=2u l=180n
M9592 t3631 t3629 vdd vdd pch w=2u l=180n
CT3634 t3634 0 0.1f
M9593 t3631 nw1162 t3634 0 nch w=1u l=180n
M9594 t3634 t3629 0 0 nch w=1u l=180n
M9595 nw1164 t3630 vdd vdd pch w=2u l=180n
M9596 nw1164 t3631 vdd vdd pch w=2u l=180n
CT3635 t3635 0 0.1f
M9597 nw1164 t3630 t3635 0 nch w=1u l=180n
M9598 t3635 t3631 0 0 nch w=1u l=180n
Cnw1164 nw1164 0 2f
M9599 nw1165 nw206 vdd vdd pch w=2u l=180n
M9600 nw1165 nw1092 vdd vdd pch w=2u l=180n
CT3636 t3636 0 0.1f
M9601 nw1165 nw206 t3636 0 nch w=1u l=180n
M9602 t3636 nw1092 0 0 nch w=1u l=180n
Cnw1165 nw1165 0 2f
M9603 nw1166 nw1163 vdd vdd pch w=2u l=180n
M9604 nw1166 nw1162 vdd vdd pch w=2u l=180n
CT3637 t3637 0 0.1f
M9605 nw1166 nw1163 t3637 0 nch w=1u l=180n
M9606 t3637 nw1162 0 0 nch w=1u l=180n
Cnw1166 nw1166 0 2f
M9607 nw1167 nw1165 vdd vdd pch w=2u l=180n
M9608 nw1167 nw1166 vdd vdd pch w=2u l=180n
CT3638 t3638 0 0.1f
M9609 nw1167 nw1165 t3638 0 nch w=1u l=180n
M9610 t3638 nw1166 0 0 nch w=1u l=180n
Cnw1167 nw1167 0 2f
CT3639 t3639 0 0.1f
CT3640 t3640 0 0.1f
CT3641 t3641 0 0.1f
M9611 t3639 nw207 vdd vdd pch w=2u l=180n
M9612 t3639 nw1097 vdd vdd pch w=2u l=180n
CT3642 t3642 0 0.1f
M9613 t3639 nw207 t3642 0 nch w=1u l=180n
M9614 t3642 nw1097 0 0 nch w=1u l=180n
M9615 t3640 nw207 vdd vdd pch w=2u l=180n
M9616 t3640 t3639 vdd vdd pch w=2u l=180n
CT3643 t3643 0 0.1f
M9617 t3640 nw207 t3643 0 nch w=1u l=180n
M9618 t3643 t3639 0 0 nch w=1u l=180n
M9619 t3641 nw1097 vdd vdd pch w=2u l=180n
M9620 t3641 t3639 vdd vdd pch w=2u l=180n
CT3644 t3644 0 0.1f
M9621 t3641 nw1097 t3644 0 nch w=1u l=180n
M9622 t3644 t3639 0 0 nch w=1u l=180n
M9623 nw1168 t3640 vdd vdd pch w=2u l=180n
M9624 nw1168 t3641 vdd vdd pch w=2u l=180n
CT3645 t3645 0 0.1f
M9625 nw1168 t3640 t3645 0 nch w=1u l=180n
M9626 t3645 t3641 0 0 nch w=1u l=180n
Cnw1168 nw1168 0 2f
CT3646 t3646 0 0.1f
CT3647 t3647 0 0.1f
CT3648 t3648 0 0.1f
M9627 t3646 nw1168 vdd vdd pch w=2u l=180n
M9628 t3646 nw1167 vdd vdd pch w=2u l=180n
CT3649 t3649 0 0.1f
M9629 t3646 nw1168 t3649 0 nch w=1u l=180n
M9630 t3649 nw1167 0 0 nch w=1u l=180n
M9631 t3647 nw1168 vdd vdd pch w=2u l=180n
M9632 t3647 t3646 vdd vdd pch w=2u l=180n
CT3650 t3650 0 0.1f
M9633 t3647 nw1168 t3650 0 nch w=1u l=180n
M9634 t3650 t3646 0 0 nch w=1u l=180n
M9635 t3648 nw1167 vdd vdd pch w=2u l=180n
M9636 t3648 t3646 vdd vdd pch w=2u l=180n
CT3651 t3651 0 0.1f
M9637 t3648 nw1167 t3651 0 nch w=1u l=180n
M9638 t3651 t3646 0 0 nch w=1u l=180n
M9639 nw1169 t3647 vdd vdd pch w=2u l=180n
M9640 nw1169 t3648 vdd vdd pch w=2u l=180n
CT3652 t3652 0 0.1f
M9641 nw1169 t3647 t3652 0 nch w=1u l=180n
M9642 t3652 t3648 0 0 nch w=1u l=180n
Cnw1169 nw1169 0 2f
M9643 nw1170 nw207 vdd vdd pch w=2u l=180n
M9644 nw1170 nw1097 vdd vdd pch w=2u l=180n
CT3653 t3653 0 0.1f
M9645 nw1170 nw207 t3653 0 nch w=1u l=180n
M9646 t3653 nw1097 0 0 nch w=1u l=180n
Cnw1170 nw1170 0 2f
M9647 nw1171 nw1168 vdd vdd pch w=2u l=180n
M9648 nw1171 nw1167 vdd vdd pch w=2u l=180n
CT3654 t3654 0 0.1f
M9649 nw1171 nw1168 t3654 0 nch w=1u l=180n
M9650 t3654 nw1167 0 0 nch w=1u l=180n
Cnw1171 nw1171 0 2f
M9651 nw1172 nw1170 vdd vdd pch w=2u l=180n
M9652 nw1172 nw1171 vdd vdd pch w=2u l=180n
CT3655 t3655 0 0.1f
M9653 nw1172 nw1170 t3655 0 nch w=1u l=180n
M9654 t3655 nw1171 0 0 nch w=1u l=180n
Cnw1172 nw1172 0 2f
CT3656 t3656 0 0.1f
CT3657 t3657 0 0.1f
CT3658 t3658 0 0.1f
M9655 t3656 nw208 vdd vdd pch w=2u l=180n
M9656 t3656 nw1100 vdd vdd pch w=2u l=180n
CT3659 t3659 0 0.1f
M9657 t3656 nw208 t3659 0 nch w=1u l=180n
M9658 t3659 nw1100 0 0 nch w=1u l=180n
M9659 t3657 nw208 vdd vdd pch w=2u l=180n
M9660 t3657 t3656 vdd vdd pch w=2u l=180n
CT3660 t3660 0 0.1f
M9661 t3657 nw208 t3660 0 nch w=1u l=180n
M9662 t3660 t3656 0 0 nch w=1u l=180n
M9663 t3658 nw1100 vdd vdd pch w=2u l=180n
M9664 t3658 t3656 vdd vdd pch w=2u l=180n
CT3661 t3661 0 0.1f
M9665 t3658 nw1100 t3661 0 nch w=1u l=180n
M9666 t3661 t3656 0 0 nch w=1u l=180n
M9667 nw1173 t3657 vdd vdd pch w=2u l=180n
M9668 nw1173 t3658 vdd vdd pch w=2u l=180n
CT3662 t3662 0 0.1f
M9669 nw1173 t3657 t3662 0 nch w=1u l=180n
M9670 t3662 t3658 0 0 nch w=1u l=180n
Cnw1173 nw1173 0 2f
CT3663 t3663 0 0.1f
CT3664 t3664 0 0.1f
CT3665 t3665 0 0.1f
M9671 t3663 nw1173 vdd vdd pch w=2u l=180n
M9672 t3663 nw1172 vdd vdd pch w=2u l=180n
CT3666 t3666 0 0.1f
M9673 t3663 nw1173 t3666 0 nch w=1u l=180n
M9674 t3666 nw1172 0 0 nch w=1u l=180n
M9675 t3664 nw1173 vdd vdd pch w=2u l=180n
M9676 t3664 t3663 vdd vdd pch w=2u l=180n
CT3667 t3667 0 0.1f
M9677 t3664 nw1173 t3667 0 nch w=1u l=180n
M9678 t3667 t3663 0 0 nch w=1u l=180n
M9679 t3665 nw1172 vdd vdd pch w=2u l=180n
M9680 t3665 t3663 vdd vdd pch w=2u l=180n
CT3668 t3668 0 0.1f
M9681 t3665 nw1172 t3668 0 nch w=1u l=180n
M9682 t3668 t3663 0 0 nch w=1u l=180n
M9683 nw1174 t3664 vdd vdd pch w=2u l=180n
M9684 nw1174 t3665 vdd vdd pch w=2u l=180n
CT3669 t3669 0 0.1f
M9685 nw1174 t3664 t3669 0 nch w=1u l=180n
M9686 t3669 t3665 0 0 nch w=1u l=180n
Cnw1174 nw1174 0 2f
M9687 nw1175 nw208 vdd vdd pch w=2u l=180n
M9688 nw1175 nw1100 vdd vdd pch w=2u l=180n
CT3670 t3670 0 0.1f
M9689 nw1175 nw208 t3670 0 nch w=1u l=180n
M9690 t3670 nw1100 0 0 nch w=1u l=180n
Cnw1175 nw1175 0 2f
M9691 nw1176 nw1173 vdd vdd pch w=2u l=180n
M9692 nw1176 nw1172 vdd vdd pch w=2u l=180n
CT3671 t3671 0 0.1f
M9693 nw1176 nw1173 t3671 0 nch w=1u l=180n
M9694 t3671 nw1172 0 0 nch w=1u l=180n
Cnw1176 nw1176 0 2f
M9695 nw1177 nw1175 vdd vdd pch w=2u l=180n
M9696 nw1177 nw1176 vdd vdd pch w=2u l=180n
CT3672 t3672 0 0.1f
M9697 nw1177 nw1175 t3672 0 nch w=1u l=180n
M9698 t3672 nw1176 0 0 nch w=1u l=180n
Cnw1177 nw1177 0 2f
CT3673 t3673 0 0.1f
CT3674 t3674 0 0.1f
CT3675 t3675 0 0.1f
M9699 t3673 nw209 vdd vdd pch w=2u l=180n
M9700 t3673 nw1104 vdd vdd pch w=2u l=180n
CT3676 t3676 0 0.1f
M9701 t3673 nw209 t3676 0 nch w=1u l=180n
M9702 t3676 nw1104 0 0 nch w=1u l=180n
M9703 t3674 nw209 vdd vdd pch w=2u l=180n
M9704 t3674 t3673 vdd vdd pch w=2u l=180n
CT3677 t3677 0 0.1f
M9705 t3674 nw209 t3677 0 nch w=1u l=180n
M9706 t3677 t3673 0 0 nch w=1u l=180n
M9707 t3675 nw1104 vdd vdd pch w=2u l=180n
M9708 t3675 t3673 vdd vdd pch w=2u l=180n
CT3678 t3678 0 0.1f
M9709 t3675 nw1104 t3678 0 nch w=1u l=180n
M9710 t3678 t3673 0 0 nch w=1u l=180n
M9711 nw1178 t3674 vdd vdd pch w=2u l=180n
M9712 nw1178 t3675 vdd vdd pch w=2u l=180n
CT3679 t3679 0 0.1f
M9713 nw1178 t3674 t3679 0 nch w=1u l=180n
M9714 t3679 t3675 0 0 nch w=1u l=180n
Cnw1178 nw1178 0 2f
CT3680 t3680 0 0.1f
M9715 t3680 nw209 vdd vdd pch w=2u l=180n
M9716 t3680 nw1104 vdd vdd pch w=2u l=180n
CT3681 t3681 0 0.1f
M9717 t3680 nw209 t3681 0 nch w=1u l=180n
M9718 t3681 nw1104 0 0 nch w=1u l=180n
M9719 nw1179 t3680 vdd vdd pch w=2u l=180n
M9720 nw1179 t3680 0 0 nch w=1u l=180n
Cnw1179 nw1179 0 2f
CT3682 t3682 0 0.1f
CT3683 t3683 0 0.1f
CT3684 t3684 0 0.1f
M9721 t3682 nw210 vdd vdd pch w=2u l=180n
M9722 t3682 nw1109 vdd vdd pch w=2u l=180n
CT3685 t3685 0 0.1f
M9723 t3682 nw210 t3685 0 nch w=1u l=180n
M9724 t3685 nw1109 0 0 nch w=1u l=180n
M9725 t3683 nw210 vdd vdd pch w=2u l=180n
M9726 t3683 t3682 vdd vdd pch w=2u l=180n
CT3686 t3686 0 0.1f
M9727 t3683 nw210 t3686 0 nch w=1u l=180n
M9728 t3686 t3682 0 0 nch w=1u l=180n
M9729 t3684 nw1109 vdd vdd pch w=2u l=180n
M9730 t3684 t3682 vdd vdd pch w=2u l=180n
CT3687 t3687 0 0.1f
M9731 t3684 nw1109 t3687 0 nch w=1u l=180n
M9732 t3687 t3682 0 0 nch w=1u l=180n
M9733 nw1180 t3683 vdd vdd pch w=2u l=180n
M9734 nw1180 t3684 vdd vdd pch w=2u l=180n
CT3688 t3688 0 0.1f
M9735 nw1180 t3683 t3688 0 nch w=1u l=180n
M9736 t3688 t3684 0 0 nch w=1u l=180n
Cnw1180 nw1180 0 2f
CT3689 t3689 0 0.1f
CT3690 t3690 0 0.1f
CT3691 t3691 0 0.1f
M9737 t3689 nw1180 vdd vdd pch w=2u l=180n
M9738 t3689 nw1179 vdd vdd pch w=2u l=180n
CT3692 t3692 0 0.1f
M9739 t3689 nw1180 t3692 0 nch w=1u l=180n
M9740 t3692 nw1179 0 0 nch w=1u l=180n
M9741 t3690 nw1180 vdd vdd pch w=2u l=180n
M9742 t3690 t3689 vdd vdd pch w=2u l=180n
CT3693 t3693 0 0.1f
M9743 t3690 nw1180 t3693 0 nch w=1u l=180n
M9744 t3693 t3689 0 0 nch w=1u l=180n
M9745 t3691 nw1179 vdd vdd pch w=2u l=180n
M9746 t3691 t3689 vdd vdd pch w=2u l=180n
CT3694 t3694 0 0.1f
M9747 t3691 nw1179 t3694 0 nch w=1u l=180n
M9748 t3694 t3689 0 0 nch w=1u l=180n
M9749 nw1181 t3690 vdd vdd pch w=2u l=180n
M9750 nw1181 t3691 vdd vdd pch w=2u l=180n
CT3695 t3695 0 0.1f
M9751 nw1181 t3690 t3695 0 nch w=1u l=180n
M9752 t3695 t3691 0 0 nch w=1u l=180n
Cnw1181 nw1181 0 2f
M9753 nw1182 nw210 vdd vdd pch w=2u l=180n
M9754 nw1182 nw1109 vdd vdd pch w=2u l=180n
CT3696 t3696 0 0.1f
M9755 nw1182 nw210 t3696 0 nch w=1u l=180n
M9756 t3696 nw1109 0 0 nch w=1u l=180n
Cnw1182 nw1182 0 2f
M9757 nw1183 nw1180 vdd vdd pch w=2u l=180n
M9758 nw1183 nw1179 vdd vdd pch w=2u l=180n
CT3697 t3697 0 0.1f
M9759 nw1183 nw1180 t3697 0 nch w=1u l=180n
M9760 t3697 nw1179 0 0 nch w=1u l=180n
Cnw1183 nw1183 0 2f
M9761 nw1184 nw1182 vdd vdd pch w=2u l=180n
M9762 nw1184 nw1183 vdd vdd pch w=2u l=180n
CT3698 t3698 0 0.1f
M9763 nw1184 nw1182 t3698 0 nch w=1u l=180n
M9764 t3698 nw1183 0 0 nch w=1u l=180n
Cnw1184 nw1184 0 2f
CT3699 t3699 0 0.1f
CT3700 t3700 0 0.1f
CT3701 t3701 0 0.1f
M9765 t3699 nw211 vdd vdd pch w=2u l=180n
M9766 t3699 nw1114 vdd vdd pch w=2u l=180n
CT3702 t3702 0 0.1f
M9767 t3699 nw211 t3702 0 nch w=1u l=180n
M9768 t3702 nw1114 0 0 nch w=1u l=180n
M9769 t3700 nw211 vdd vdd pch w=2u l=180n
M9770 t3700 t3699 vdd vdd pch w=2u l=180n
CT3703 t3703 0 0.1f
M9771 t3700 nw211 t3703 0 nch w=1u l=180n
M9772 t3703 t3699 0 0 nch w=1u l=180n
M9773 t3701 nw1114 vdd vdd pch w=2u l=180n
M9774 t3701 t3699 vdd vdd pch w=2u l=180n
CT3704 t3704 0 0.1f
M9775 t3701 nw1114 t3704 0 nch w=1u l=180n
M9776 t3704 t3699 0 0 nch w=1u l=180n
M9777 nw1185 t3700 vdd vdd pch w=2u l=180n
M9778 nw1185 t3701 vdd vdd pch w=2u l=180n
CT3705 t3705 0 0.1f
M9779 nw1185 t3700 t3705 0 nch w=1u l=180n
M9780 t3705 t3701 0 0 nch w=1u l=180n
Cnw1185 nw1185 0 2f
CT3706 t3706 0 0.1f
CT3707 t3707 0 0.1f
CT3708 t3708 0 0.1f
M9781 t3706 nw1185 vdd vdd pch w=2u l=180n
M9782 t3706 nw1184 vdd vdd pch w=2u l=180n
CT3709 t3709 0 0.1f
M9783 t3706 nw1185 t3709 0 nch w=1u l=180n
M9784 t3709 nw1184 0 0 nch w=1u l=180n
M9785 t3707 nw1185 vdd vdd pch w=2u l=180n
M9786 t3707 t3706 vdd vdd pch w=2u l=180n
CT3710 t3710 0 0.1f
M9787 t3707 nw1185 t3710 0 nch w=1u l=180n
M9788 t3710 t3706 0 0 nch w=1u l=180n
M9789 t3708 nw1184 vdd vdd pch w=2u l=180n
M9790 t3708 t3706 vdd vdd pch w=2u l=180n
CT3711 t3711 0 0.1f
M9791 t3708 nw1184 t3711 0 nch w=1u l=180n
M9792 t3711 t3706 0 0 nch w=1u l=180n
M9793 nw1186 t3707 vdd vdd pch w=2u l=180n
M9794 nw1186 t3708 vdd vdd pch w=2u l=180n
CT3712 t3712 0 0.1f
M9795 nw1186 t3707 t3712 0 nch w=1u l=180n
M9796 t3712 t3708 0 0 nch w=1u l=180n
Cnw1186 nw1186 0 2f
M9797 nw1187 nw211 vdd vdd pch w=2u l=180n
M9798 nw1187 nw1114 vdd vdd pch w=2u l=180n
CT3713 t3713 0 0.1f
M9799 nw1187 nw211 t3713 0 nch w=1u l=180n
M9800 t3713 nw1114 0 0 nch w=1u l=180n
Cnw1187 nw1187 0 2f
M9801 nw1188 nw1185 vdd vdd pch w=2u l=180n
M9802 nw1188 nw1184 vdd vdd pch w=2u l=180n
CT3714 t3714 0 0.1f
M9803 nw1188 nw1185 t3714 0 nch w=1u l=180n
M9804 t3714 nw1184 0 0 nch w=1u l=180n
Cnw1188 nw1188 0 2f
M9805 nw1189 nw1187 vdd vdd pch w=2u l=180n
M9806 nw1189 nw1188 vdd vdd pch w=2u l=180n
CT3715 t3715 0 0.1f
M9807 nw1189 nw1187 t3715 0 nch w=1u l=180n
M9808 t3715 nw1188 0 0 nch w=1u l=180n
Cnw1189 nw1189 0 2f
CT3716 t3716 0 0.1f
CT3717 t3717 0 0.1f
CT3718 t3718 0 0.1f
M9809 t3716 nw212 vdd vdd pch w=2u l=180n
M9810 t3716 nw1119 vdd vdd pch w=2u l=180n
CT3719 t3719 0 0.1f
M9811 t3716 nw212 t3719 0 nch w=1u l=180n
M9812 t3719 nw1119 0 0 nch w=1u l=180n
M9813 t3717 nw212 vdd vdd pch w=2u l=180n
M9814 t3717 t3716 vdd vdd pch w=2u l=180n
CT3720 t3720 0 0.1f
M9815 t3717 nw212 t3720 0 nch w=1u l=180n
M9816 t3720 t3716 0 0 nch w=1u l=180n
M9817 t3718 nw1119 vdd vdd pch w=2u l=180n
M9818 t3718 t3716 vdd vdd pch w=2u l=180n
CT3721 t3721 0 0.1f
M9819 t3718 nw1119 t3721 0 nch w=1u l=180n
M9820 t3721 t3716 0 0 nch w=1u l=180n
M9821 nw1190 t3717 vdd vdd pch w=2u l=180n
M9822 nw1190 t3718 vdd vdd pch w=2u l=180n
CT3722 t3722 0 0.1f
M9823 nw1190 t3717 t3722 0 nch w=1u l=180n
M9824 t3722 t3718 0 0 nch w=1u l=180n
Cnw1190 nw1190 0 2f
CT3723 t3723 0 0.1f
CT3724 t3724 0 0.1f
CT3725 t3725 0 0.1f
M9825 t3723 nw1190 vdd vdd pch w=2u l=180n
M9826 t3723 nw1189 vdd vdd pch w=2u l=180n
CT3726 t3726 0 0.1f
M9827 t3723 nw1190 t3726 0 nch w=1u l=180n
M9828 t3726 nw1189 0 0 nch w=1u l=180n
M9829 t3724 nw1190 vdd vdd pch w=2u l=180n
M9830 t3724 t3723 vdd vdd pch w=2u l=180n
CT3727 t3727 0 0.1f
M9831 t3724 nw1190 t3727 0 nch w=1u l=180n
M9832 t3727 t3723 0 0 nch w=1u l=180n
M9833 t3725 nw1189 vdd vdd pch w=2u l=180n
M9834 t3725 t3723 vdd vdd pch w=2u l=180n
CT3728 t3728 0 0.1f
M9835 t3725 nw1189 t3728 0 nch w=1u l=180n
M9836 t3728 t3723 0 0 nch w=1u l=180n
M9837 nw1191 t3724 vdd vdd pch w=2u l=180n
M9838 nw1191 t3725 vdd vdd pch w=2u l=180n
CT3729 t3729 0 0.1f
M9839 nw1191 t3724 t3729 0 nch w=1u l=180n
M9840 t3729 t3725 0 0 nch w=1u l=180n
Cnw1191 nw1191 0 2f
M9841 nw1192 nw212 vdd vdd pch w=2u l=180n
M9842 nw1192 nw1119 vdd vdd pch w=2u l=180n
CT3730 t3730 0 0.1f
M9843 nw1192 nw212 t3730 0 nch w=1u l=180n
M9844 t3730 nw1119 0 0 nch w=1u l=180n
Cnw1192 nw1192 0 2f
M9845 nw1193 nw1190 vdd vdd pch w=2u l=180n
M9846 nw1193 nw1189 vdd vdd pch w=2u l=180n
CT3731 t3731 0 0.1f
M9847 nw1193 nw1190 t3731 0 nch w=1u l=180n
M9848 t3731 nw1189 0 0 nch w=1u l=180n
Cnw1193 nw1193 0 2f
M9849 nw1194 nw1192 vdd vdd pch w=2u l=180n
M9850 nw1194 nw1193 vdd vdd pch w=2u l=180n
CT3732 t3732 0 0.1f
M9851 nw1194 nw1192 t3732 0 nch w=1u l=180n
M9852 t3732 nw1193 0 0 nch w=1u l=180n
Cnw1194 nw1194 0 2f
CT3733 t3733 0 0.1f
CT3734 t3734 0 0.1f
CT3735 t3735 0 0.1f
M9853 t3733 nw213 vdd vdd pch w=2u l=180n
M9854 t3733 nw1124 vdd vdd pch w=2u l=180n
CT3736 t3736 0 0.1f
M9855 t3733 nw213 t3736 0 nch w=1u l=180n
M9856 t3736 nw1124 0 0 nch w=1u l=180n
M9857 t3734 nw213 vdd vdd pch w=2u l=180n
M9858 t3734 t3733 vdd vdd pch w=2u l=180n
CT3737 t3737 0 0.1f
M9859 t3734 nw213 t3737 0 nch w=1u l=180n
M9860 t3737 t3733 0 0 nch w=1u l=180n
M9861 t3735 nw1124 vdd vdd pch w=2u l=180n
M9862 t3735 t3733 vdd vdd pch w=2u l=180n
CT3738 t3738 0 0.1f
M9863 t3735 nw1124 t3738 0 nch w=1u l=180n
M9864 t3738 t3733 0 0 nch w=1u l=180n
M9865 nw1195 t3734 vdd vdd pch w=2u l=180n
M9866 nw1195 t3735 vdd vdd pch w=2u l=180n
CT3739 t3739 0 0.1f
M9867 nw1195 t3734 t3739 0 nch w=1u l=180n
M9868 t3739 t3735 0 0 nch w=1u l=180n
Cnw1195 nw1195 0 2f
CT3740 t3740 0 0.1f
CT3741 t3741 0 0.1f
CT3742 t3742 0 0.1f
M9869 t3740 nw1195 vdd vdd pch w=2u l=180n
M9870 t3740 nw1194 vdd vdd pch w=2u l=180n
CT3743 t3743 0 0.1f
M9871 t3740 nw1195 t3743 0 nch w=1u l=180n
M9872 t3743 nw1194 0 0 nch w=1u l=180n
M9873 t3741 nw1195 vdd vdd pch w=2u l=180n
M9874 t3741 t3740 vdd vdd pch w=2u l=180n
CT3744 t3744 0 0.1f
M9875 t3741 nw1195 t3744 0 nch w=1u l=180n
M9876 t3744 t3740 0 0 nch w=1u l=180n
M9877 t3742 nw1194 vdd vdd pch w=2u l=180n
M9878 t3742 t3740 vdd vdd pch w=2u l=180n
CT3745 t3745 0 0.1f
M9879 t3742 nw1194 t3745 0 nch w=1u l=180n
M9880 t3745 t3740 0 0 nch w=1u l=180n
M9881 nw1196 t3741 vdd vdd pch w=2u l=180n
M9882 nw1196 t3742 vdd vdd pch w=2u l=180n
CT3746 t3746 0 0.1f
M9883 nw1196 t3741 t3746 0 nch w=1u l=180n
M9884 t3746 t3742 0 0 nch w=1u l=180n
Cnw1196 nw1196 0 2f
M9885 nw1197 nw213 vdd vdd pch w=2u l=180n
M9886 nw1197 nw1124 vdd vdd pch w=2u l=180n
CT3747 t3747 0 0.1f
M9887 nw1197 nw213 t3747 0 nch w=1u l=180n
M9888 t3747 nw1124 0 0 nch w=1u l=180n
Cnw1197 nw1197 0 2f
M9889 nw1198 nw1195 vdd vdd pch w=2u l=180n
M9890 nw1198 nw1194 vdd vdd pch w=2u l=180n
CT3748 t3748 0 0.1f
M9891 nw1198 nw1195 t3748 0 nch w=1u l=180n
M9892 t3748 nw1194 0 0 nch w=1u l=180n
Cnw1198 nw1198 0 2f
M9893 nw1199 nw1197 vdd vdd pch w=2u l=180n
M9894 nw1199 nw1198 vdd vdd pch w=2u l=180n
CT3749 t3749 0 0.1f
M9895 nw1199 nw1197 t3749 0 nch w=1u l=180n
M9896 t3749 nw1198 0 0 nch w=1u l=180n
Cnw1199 nw1199 0 2f
CT3750 t3750 0 0.1f
CT3751 t3751 0 0.1f
CT3752 t3752 0 0.1f
M9897 t3750 nw214 vdd vdd pch w=2u l=180n
M9898 t3750 nw1129 vdd vdd pch w=2u l=180n
CT3753 t3753 0 0.1f
M9899 t3750 nw214 t3753 0 nch w=1u l=180n
M9900 t3753 nw1129 0 0 nch w=1u l=180n
M9901 t3751 nw214 vdd vdd pch w=2u l=180n
M9902 t3751 t3750 vdd vdd pch w=2u l=180n
CT3754 t3754 0 0.1f
M9903 t3751 nw214 t3754 0 nch w=1u l=180n
M9904 t3754 t3750 0 0 nch w=1u l=180n
M9905 t3752 nw1129 vdd vdd pch w=2u l=180n
M9906 t3752 t3750 vdd vdd pch w=2u l=180n
CT3755 t3755 0 0.1f
M9907 t3752 nw1129 t3755 0 nch w=1u l=180n
M9908 t3755 t3750 0 0 nch w=1u l=180n
M9909 nw1200 t3751 vdd vdd pch w=2u l=180n
M9910 nw1200 t3752 vdd vdd pch w=2u l=180n
CT3756 t3756 0 0.1f
M9911 nw1200 t3751 t3756 0 nch w=1u l=180n
M9912 t3756 t3752 0 0 nch w=1u l=180n
Cnw1200 nw1200 0 2f
CT3757 t3757 0 0.1f
CT3758 t3758 0 0.1f
CT3759 t3759 0 0.1f
M9913 t3757 nw1200 vdd vdd pch w=2u l=180n
M9914 t3757 nw1199 vdd vdd pch w=2u l=180n
CT3760 t3760 0 0.1f
M9915 t3757 nw1200 t3760 0 nch w=1u l=180n
M9916 t3760 nw1199 0 0 nch w=1u l=180n
M9917 t3758 nw1200 vdd vdd pch w=2u l=180n
M9918 t3758 t3757 vdd vdd pch w=2u l=180n
CT3761 t3761 0 0.1f
M9919 t3758 nw1200 t3761 0 nch w=1u l=180n
M9920 t3761 t3757 0 0 nch w=1u l=180n
M9921 t3759 nw1199 vdd vdd pch w=2u l=180n
M9922 t3759 t3757 vdd vdd pch w=2u l=180n
CT3762 t3762 0 0.1f
M9923 t3759 nw1199 t3762 0 nch w=1u l=180n
M9924 t3762 t3757 0 0 nch w=1u l=180n
M9925 nw1201 t3758 vdd vdd pch w=2u l=180n
M9926 nw1201 t3759 vdd vdd pch w=2u l=180n
CT3763 t3763 0 0.1f
M9927 nw1201 t3758 t3763 0 nch w=1u l=180n
M9928 t3763 t3759 0 0 nch w=1u l=180n
Cnw1201 nw1201 0 2f
M9929 nw1202 nw214 vdd vdd pch w=2u l=180n
M9930 nw1202 nw1129 vdd vdd pch w=2u l=180n
CT3764 t3764 0 0.1f
M9931 nw1202 nw214 t3764 0 nch w=1u l=180n
M9932 t3764 nw1129 0 0 nch w=1u l=180n
Cnw1202 nw1202 0 2f
M9933 nw1203 nw1200 vdd vdd pch w=2u l=180n
M9934 nw1203 nw1199 vdd vdd pch w=2u l=180n
CT3765 t3765 0 0.1f
M9935 nw1203 nw1200 t3765 0 nch w=1u l=180n
M9936 t3765 nw1199 0 0 nch w=1u l=180n
Cnw1203 nw1203 0 2f
M9937 nw1204 nw1202 vdd vdd pch w=2u l=180n
M9938 nw1204 nw1203 vdd vdd pch w=2u l=180n
CT3766 t3766 0 0.1f
M9939 nw1204 nw1202 t3766 0 nch w=1u l=180n
M9940 t3766 nw1203 0 0 nch w=1u l=180n
Cnw1204 nw1204 0 2f
CT3767 t3767 0 0.1f
CT3768 t3768 0 0.1f
CT3769 t3769 0 0.1f
M9941 t3767 nw215 vdd vdd pch w=2u l=180n
M9942 t3767 nw1134 vdd vdd pch w=2u l=180n
CT3770 t3770 0 0.1f
M9943 t3767 nw215 t3770 0 nch w=1u l=180n
M9944 t3770 nw1134 0 0 nch w=1u l=180n
M9945 t3768 nw215 vdd vdd pch w=2u l=180n
M9946 t3768 t3767 vdd vdd pch w=2u l=180n
CT3771 t3771 0 0.1f
M9947 t3768 nw215 t3771 0 nch w=1u l=180n
M9948 t3771 t3767 0 0 nch w=1u l=180n
M9949 t3769 nw1134 vdd vdd pch w=2u l=180n
M9950 t3769 t3767 vdd vdd pch w=2u l=180n
CT3772 t3772 0 0.1f
M9951 t3769 nw1134 t3772 0 nch w=1u l=180n
M9952 t3772 t3767 0 0 nch w=1u l=180n
M9953 nw1205 t3768 vdd vdd pch w=2u l=180n
M9954 nw1205 t3769 vdd vdd pch w=2u l=180n
CT3773 t3773 0 0.1f
M9955 nw1205 t3768 t3773 0 nch w=1u l=180n
M9956 t3773 t3769 0 0 nch w=1u l=180n
Cnw1205 nw1205 0 2f
CT3774 t3774 0 0.1f
CT3775 t3775 0 0.1f
CT3776 t3776 0 0.1f
M9957 t3774 nw1205 vdd vdd pch w=2u l=180n
M9958 t3774 nw1204 vdd vdd pch w=2u l=180n
CT3777 t3777 0 0.1f
M9959 t3774 nw1205 t3777 0 nch w=1u l=180n
M9960 t3777 nw1204 0 0 nch w=1u l=180n
M9961 t3775 nw1205 vdd vdd pch w=2u l=180n
M9962 t3775 t3774 vdd vdd pch w=2u l=180n
CT3778 t3778 0 0.1f
M9963 t3775 nw1205 t3778 0 nch w=1u l=180n
M9964 t3778 t3774 0 0 nch w=1u l=180n
M9965 t3776 nw1204 vdd vdd pch w=2u l=180n
M9966 t3776 t3774 vdd vdd pch w=2u l=180n
CT3779 t3779 0 0.1f
M9967 t3776 nw1204 t3779 0 nch w=1u l=180n
M9968 t3779 t3774 0 0 nch w=1u l=180n
M9969 nw1206 t3775 vdd vdd pch w=2u l=180n
M9970 nw1206 t3776 vdd vdd pch w=2u l=180n
CT3780 t3780 0 0.1f
M9971 nw1206 t3775 t3780 0 nch w=1u l=180n
M9972 t3780 t3776 0 0 nch w=1u l=180n
Cnw1206 nw1206 0 2f
M9973 nw1207 nw215 vdd vdd pch w=2u l=180n
M9974 nw1207 nw1134 vdd vdd pch w=2u l=180n
CT3781 t3781 0 0.1f
M9975 nw1207 nw215 t3781 0 nch w=1u l=180n
M9976 t3781 nw1134 0 0 nch w=1u l=180n
Cnw1207 nw1207 0 2f
M9977 nw1208 nw1205 vdd vdd pch w=2u l=180n
M9978 nw1208 nw1204 vdd vdd pch w=2u l=180n
CT3782 t3782 0 0.1f
M9979 nw1208 nw1205 t3782 0 nch w=1u l=180n
M9980 t3782 nw1204 0 0 nch w=1u l=180n
Cnw1208 nw1208 0 2f
M9981 nw1209 nw1207 vdd vdd pch w=2u l=180n
M9982 nw1209 nw1208 vdd vdd pch w=2u l=180n
CT3783 t3783 0 0.1f
M9983 nw1209 nw1207 t3783 0 nch w=1u l=180n
M9984 t3783 nw1208 0 0 nch w=1u l=180n
Cnw1209 nw1209 0 2f
CT3784 t3784 0 0.1f
CT3785 t3785 0 0.1f
CT3786 t3786 0 0.1f
M9985 t3784 nw216 vdd vdd pch w=2u l=180n
M9986 t3784 nw1139 vdd vdd pch w=2u l=180n
CT3787 t3787 0 0.1f
M9987 t3784 nw216 t3787 0 nch w=1u l=180n
M9988 t3787 nw1139 0 0 nch w=1u l=180n
M9989 t3785 nw216 vdd vdd pch w=2u l=180n
M9990 t3785 t3784 vdd vdd pch w=2u l=180n
CT3788 t3788 0 0.1f
M9991 t3785 nw216 t3788 0 nch w=1u l=180n
M9992 t3788 t3784 0 0 nch w=1u l=180n
M9993 t3786 nw1139 vdd vdd pch w=2u l=180n
M9994 t3786 t3784 vdd vdd pch w=2u l=180n
CT3789 t3789 0 0.1f
M9995 t3786 nw1139 t3789 0 nch w=1u l=180n
M9996 t3789 t3784 0 0 nch w=1u l=180n
M9997 nw1210 t3785 vdd vdd pch w=2u l=180n
M9998 nw1210 t3786 vdd vdd pch w=2u l=180n
CT3790 t3790 0 0.1f
M9999 nw1210 t3785 t3790 0 nch w=1u l=180n
M10000 t3790 t3786 0 0 nch w=1u l=180n
Cnw1210 nw1210 0 2f
CT3791 t3791 0 0.1f
CT3792 t3792 0 0.1f
CT3793 t3793 0 0.1f
M10001 t3791 nw1210 vdd vdd pch w=2u l=180n
M10002 t3791 nw1209 vdd vdd pch w=2u l=180n
CT3794 t3794 0 0.1f
M10003 t3791 nw1210 t3794 0 nch w=1u l=180n
M10004 t3794 nw1209 0 0 nch w=1u l=180n
M10005 t3792 nw1210 vdd vdd pch w=2u l=180n
M10006 t3792 t3791 vdd vdd pch w=2u l=180n
CT3795 t3795 0 0.1f
M10007 t3792 nw1210 t3795 0 nch w=1u l=180n
M10008 t3795 t3791 0 0 nch w=1u l=180n
M10009 t3793 nw1209 vdd vdd pch w=2u l=180n
M10010 t3793 t3791 vdd vdd pch w=2u l=180n
CT3796 t3796 0 0.1f
M10011 t3793 nw1209 t3796 0 nch w=1u l=180n
M10012 t3796 t3791 0 0 nch w=1u l=180n
M10013 nw1211 t3792 vdd vdd pch w=2u l=180n
M10014 nw1211 t3793 vdd vdd pch w=2u l=180n
CT3797 t3797 0 0.1f
M10015 nw1211 t3792 t3797 0 nch w=1u l=180n
M10016 t3797 t3793 0 0 nch w=1u l=180n
Cnw1211 nw1211 0 2f
M10017 nw1212 nw216 vdd vdd pch w=2u l=180n
M10018 nw1212 nw1139 vdd vdd pch w=2u l=180n
CT3798 t3798 0 0.1f
M10019 nw1212 nw216 t3798 0 nch w=1u l=180n
M10020 t3798 nw1139 0 0 nch w=1u l=180n
Cnw1212 nw1212 0 2f
M10021 nw1213 nw1210 vdd vdd pch w=2u l=180n
M10022 nw1213 nw1209 vdd vdd pch w=2u l=180n
CT3799 t3799 0 0.1f
M10023 nw1213 nw1210 t3799 0 nch w=1u l=180n
M10024 t3799 nw1209 0 0 nch w=1u l=180n
Cnw1213 nw1213 0 2f
M10025 nw1214 nw1212 vdd vdd pch w=2u l=180n
M10026 nw1214 nw1213 vdd vdd pch w=2u l=180n
CT3800 t3800 0 0.1f
M10027 nw1214 nw1212 t3800 0 nch w=1u l=180n
M10028 t3800 nw1213 0 0 nch w=1u l=180n
Cnw1214 nw1214 0 2f
CT3801 t3801 0 0.1f
CT3802 t3802 0 0.1f
CT3803 t3803 0 0.1f
M10029 t3801 nw217 vdd vdd pch w=2u l=180n
M10030 t3801 nw1144 vdd vdd pch w=2u l=180n
CT3804 t3804 0 0.1f
M10031 t3801 nw217 t3804 0 nch w=1u l=180n
M10032 t3804 nw1144 0 0 nch w=1u l=180n
M10033 t3802 nw217 vdd vdd pch w=2u l=180n
M10034 t3802 t3801 vdd vdd pch w=2u l=180n
CT3805 t3805 0 0.1f
M10035 t3802 nw217 t3805 0 nch w=1u l=180n
M10036 t3805 t3801 0 0 nch w=1u l=180n
M10037 t3803 nw1144 vdd vdd pch w=2u l=180n
M10038 t3803 t3801 vdd vdd pch w=2u l=180n
CT3806 t3806 0 0.1f
M10039 t3803 nw1144 t3806 0 nch w=1u l=180n
M10040 t3806 t3801 0 0 nch w=1u l=180n
M10041 nw1215 t3802 vdd vdd pch w=2u l=180n
M10042 nw1215 t3803 vdd vdd pch w=2u l=180n
CT3807 t3807 0 0.1f
M10043 nw1215 t3802 t3807 0 nch w=1u l=180n
M10044 t3807 t3803 0 0 nch w=1u l=180n
Cnw1215 nw1215 0 2f
CT3808 t3808 0 0.1f
CT3809 t3809 0 0.1f
CT3810 t3810 0 0.1f
M10045 t3808 nw1215 vdd vdd pch w=2u l=180n
M10046 t3808 nw1214 vdd vdd pch w=2u l=180n
CT3811 t3811 0 0.1f
M10047 t3808 nw1215 t3811 0 nch w=1u l=180n
M10048 t3811 nw1214 0 0 nch w=1u l=180n
M10049 t3809 nw1215 vdd vdd pch w=2u l=180n
M10050 t3809 t3808 vdd vdd pch w=2u l=180n
CT3812 t3812 0 0.1f
M10051 t3809 nw1215 t3812 0 nch w=1u l=180n
M10052 t3812 t3808 0 0 nch w=1u l=180n
M10053 t3810 nw1214 vdd vdd pch w=2u l=180n
M10054 t3810 t3808 vdd vdd pch w=2u l=180n
CT3813 t3813 0 0.1f
M10055 t3810 nw1214 t3813 0 nch w=1u l=180n
M10056 t3813 t3808 0 0 nch w=1u l=180n
M10057 nw1216 t3809 vdd vdd pch w=2u l=180n
M10058 nw1216 t3810 vdd vdd pch w=2u l=180n
CT3814 t3814 0 0.1f
M10059 nw1216 t3809 t3814 0 nch w=1u l=180n
M10060 t3814 t3810 0 0 nch w=1u l=180n
Cnw1216 nw1216 0 2f
M10061 nw1217 nw217 vdd vdd pch w=2u l=180n
M10062 nw1217 nw1144 vdd vdd pch w=2u l=180n
CT3815 t3815 0 0.1f
M10063 nw1217 nw217 t3815 0 nch w=1u l=180n
M10064 t3815 nw1144 0 0 nch w=1u l=180n
Cnw1217 nw1217 0 2f
M10065 nw1218 nw1215 vdd vdd pch w=2u l=180n
M10066 nw1218 nw1214 vdd vdd pch w=2u l=180n
CT3816 t3816 0 0.1f
M10067 nw1218 nw1215 t3816 0 nch w=1u l=180n
M10068 t3816 nw1214 0 0 nch w=1u l=180n
Cnw1218 nw1218 0 2f
M10069 nw1219 nw1217 vdd vdd pch w=2u l=180n
M10070 nw1219 nw1218 vdd vdd pch w=2u l=180n
CT3817 t3817 0 0.1f
M10071 nw1219 nw1217 t3817 0 nch w=1u l=180n
M10072 t3817 nw1218 0 0 nch w=1u l=180n
Cnw1219 nw1219 0 2f
CT3818 t3818 0 0.1f
CT3819 t3819 0 0.1f
CT3820 t3820 0 0.1f
M10073 t3818 nw218 vdd vdd pch w=2u l=180n
M10074 t3818 nw1149 vdd vdd pch w=2u l=180n
CT3821 t3821 0 0.1f
M10075 t3818 nw218 t3821 0 nch w=1u l=180n
M10076 t3821 nw1149 0 0 nch w=1u l=180n
M10077 t3819 nw218 vdd vdd pch w=2u l=180n
M10078 t3819 t3818 vdd vdd pch w=2u l=180n
CT3822 t3822 0 0.1f
M10079 t3819 nw218 t3822 0 nch w=1u l=180n
M10080 t3822 t3818 0 0 nch w=1u l=180n
M10081 t3820 nw1149 vdd vdd pch w=2u l=180n
M10082 t3820 t3818 vdd vdd pch w=2u l=180n
CT3823 t3823 0 0.1f
M10083 t3820 nw1149 t3823 0 nch w=1u l=180n
M10084 t3823 t3818 0 0 nch w=1u l=180n
M10085 nw1220 t3819 vdd vdd pch w=2u l=180n
M10086 nw1220 t3820 vdd vdd pch w=2u l=180n
CT3824 t3824 0 0.1f
M10087 nw1220 t3819 t3824 0 nch w=1u l=180n
M10088 t3824 t3820 0 0 nch w=1u l=180n
Cnw1220 nw1220 0 2f
CT3825 t3825 0 0.1f
CT3826 t3826 0 0.1f
CT3827 t3827 0 0.1f
M10089 t3825 nw1220 vdd vdd pch w=2u l=180n
M10090 t3825 nw1219 vdd vdd pch w=2u l=180n
CT3828 t3828 0 0.1f
M10091 t3825 nw1220 t3828 0 nch w=1u l=180n
M10092 t3828 nw1219 0 0 nch w=1u l=180n
M10093 t3826 nw1220 vdd vdd pch w=2u l=180n
M10094 t3826 t3825 vdd vdd pch w=2u l=180n
CT3829 t3829 0 0.1f
M10095 t3826 nw1220 t3829 0 nch w=1u l=180n
M10096 t3829 t3825 0 0 nch w=1u l=180n
M10097 t3827 nw1219 vdd vdd pch w=2u l=180n
M10098 t3827 t3825 vdd vdd pch w=2u l=180n
CT3830 t3830 0 0.1f
M10099 t3827 nw1219 t3830 0 nch w=1u l=180n
M10100 t3830 t3825 0 0 nch w=1u l=180n
M10101 nw1221 t3826 vdd vdd pch w=2u l=180n
M10102 nw1221 t3827 vdd vdd pch w=2u l=180n
CT3831 t3831 0 0.1f
M10103 nw1221 t3826 t3831 0 nch w=1u l=180n
M10104 t3831 t3827 0 0 nch w=1u l=180n
Cnw1221 nw1221 0 2f
M10105 nw1222 nw218 vdd vdd pch w=2u l=180n
M10106 nw1222 nw1149 vdd vdd pch w=2u l=180n
CT3832 t3832 0 0.1f
M10107 nw1222 nw218 t3832 0 nch w=1u l=180n
M10108 t3832 nw1149 0 0 nch w=1u l=180n
Cnw1222 nw1222 0 2f
M10109 nw1223 nw1220 vdd vdd pch w=2u l=180n
M10110 nw1223 nw1219 vdd vdd pch w=2u l=180n
CT3833 t3833 0 0.1f
M10111 nw1223 nw1220 t3833 0 nch w=1u l=180n
M10112 t3833 nw1219 0 0 nch w=1u l=180n
Cnw1223 nw1223 0 2f
M10113 nw1224 nw1222 vdd vdd pch w=2u l=180n
M10114 nw1224 nw1223 vdd vdd pch w=2u l=180n
CT3834 t3834 0 0.1f
M10115 nw1224 nw1222 t3834 0 nch w=1u l=180n
M10116 t3834 nw1223 0 0 nch w=1u l=180n
Cnw1224 nw1224 0 2f
CT3835 t3835 0 0.1f
CT3836 t3836 0 0.1f
CT3837 t3837 0 0.1f
M10117 t3835 nw219 vdd vdd pch w=2u l=180n
M10118 t3835 nw1154 vdd vdd pch w=2u l=180n
CT3838 t3838 0 0.1f
M10119 t3835 nw219 t3838 0 nch w=1u l=180n
M10120 t3838 nw1154 0 0 nch w=1u l=180n
M10121 t3836 nw219 vdd vdd pch w=2u l=180n
M10122 t3836 t3835 vdd vdd pch w=2u l=180n
CT3839 t3839 0 0.1f
M10123 t3836 nw219 t3839 0 nch w=1u l=180n
M10124 t3839 t3835 0 0 nch w=1u l=180n
M10125 t3837 nw1154 vdd vdd pch w=2u l=180n
M10126 t3837 t3835 vdd vdd pch w=2u l=180n
CT3840 t3840 0 0.1f
M10127 t3837 nw1154 t3840 0 nch w=1u l=180n
M10128 t3840 t3835 0 0 nch w=1u l=180n
M10129 nw1225 t3836 vdd vdd pch w=2u l=180n
M10130 nw1225 t3837 vdd vdd pch w=2u l=180n
CT3841 t3841 0 0.1f
M10131 nw1225 t3836 t3841 0 nch w=1u l=180n
M10132 t3841 t3837 0 0 nch w=1u l=180n
Cnw1225 nw1225 0 2f
CT3842 t3842 0 0.1f
CT3843 t3843 0 0.1f
CT3844 t3844 0 0.1f
M10133 t3842 nw1225 vdd vdd pch w=2u l=180n
M10134 t3842 nw1224 vdd vdd pch w=2u l=180n
CT3845 t3845 0 0.1f
M10135 t3842 nw1225 t3845 0 nch w=1u l=180n
M10136 t3845 nw1224 0 0 nch w=1u l=180n
M10137 t3843 nw1225 vdd vdd pch w=2u l=180n
M10138 t3843 t3842 vdd vdd pch w=2u l=180n
CT3846 t3846 0 0.1f
M10139 t3843 nw1225 t3846 0 nch w=1u l=180n
M10140 t3846 t3842 0 0 nch w=1u l=180n
M10141 t3844 nw1224 vdd vdd pch w=2u l=180n
M10142 t3844 t3842 vdd vdd pch w=2u l=180n
CT3847 t3847 0 0.1f
M10143 t3844 nw1224 t3847 0 nch w=1u l=180n
M10144 t3847 t3842 0 0 nch w=1u l=180n
M10145 nw1226 t3843 vdd vdd pch w=2u l=180n
M10146 nw1226 t3844 vdd vdd pch w=2u l=180n
CT3848 t3848 0 0.1f
M10147 nw1226 t3843 t3848 0 nch w=1u l=180n
M10148 t3848 t3844 0 0 nch w=1u l=180n
Cnw1226 nw1226 0 2f
M10149 nw1227 nw219 vdd vdd pch w=2u l=180n
M10150 nw1227 nw1154 vdd vdd pch w=2u l=180n
CT3849 t3849 0 0.1f
M10151 nw1227 nw219 t3849 0 nch w=1u l=180n
M10152 t3849 nw1154 0 0 nch w=1u l=180n
Cnw1227 nw1227 0 2f
M10153 nw1228 nw1225 vdd vdd pch w=2u l=180n
M10154 nw1228 nw1224 vdd vdd pch w=2u l=180n
CT3850 t3850 0 0.1f
M10155 nw1228 nw1225 t3850 0 nch w=1u l=180n
M10156 t3850 nw1224 0 0 nch w=1u l=180n
Cnw1228 nw1228 0 2f
M10157 nw1229 nw1227 vdd vdd pch w=2u l=180n
M10158 nw1229 nw1228 vdd vdd pch w=2u l=180n
CT3851 t3851 0 0.1f
M10159 nw1229 nw1227 t3851 0 nch w=1u l=180n
M10160 t3851 nw1228 0 0 nch w=1u l=180n
Cnw1229 nw1229 0 2f
CT3852 t3852 0 0.1f
CT3853 t3853 0 0.1f
CT3854 t3854 0 0.1f
M10161 t3852 nw220 vdd vdd pch w=2u l=180n
M10162 t3852 nw1159 vdd vdd pch w=2u l=180n
CT3855 t3855 0 0.1f
M10163 t3852 nw220 t3855 0 nch w=1u l=180n
M10164 t3855 nw1159 0 0 nch w=1u l=180n
M10165 t3853 nw220 vdd vdd pch w=2u l=180n
M10166 t3853 t3852 vdd vdd pch w=2u l=180n
CT3856 t3856 0 0.1f
M10167 t3853 nw220 t3856 0 nch w=1u l=180n
M10168 t3856 t3852 0 0 nch w=1u l=180n
M10169 t3854 nw1159 vdd vdd pch w=2u l=180n
M10170 t3854 t3852 vdd vdd pch w=2u l=180n
CT3857 t3857 0 0.1f
M10171 t3854 nw1159 t3857 0 nch w=1u l=180n
M10172 t3857 t3852 0 0 nch w=1u l=180n
M10173 nw1230 t3853 vdd vdd pch w=2u l=180n
M10174 nw1230 t3854 vdd vdd pch w=2u l=180n
CT3858 t3858 0 0.1f
M10175 nw1230 t3853 t3858 0 nch w=1u l=180n
M10176 t3858 t3854 0 0 nch w=1u l=180n
Cnw1230 nw1230 0 2f
CT3859 t3859 0 0.1f
CT3860 t3860 0 0.1f
CT3861 t3861 0 0.1f
M10177 t3859 nw1230 vdd vdd pch w=2u l=180n
M10178 t3859 nw1229 vdd vdd pch w=2u l=180n
CT3862 t3862 0 0.1f
M10179 t3859 nw1230 t3862 0 nch w=1u l=180n
M10180 t3862 nw1229 0 0 nch w=1u l=180n
M10181 t3860 nw1230 vdd vdd pch w=2u l=180n
M10182 t3860 t3859 vdd vdd pch w=2u l=180n
CT3863 t3863 0 0.1f
M10183 t3860 nw1230 t3863 0 nch w=1u l=180n
M10184 t3863 t3859 0 0 nch w=1u l=180n
M10185 t3861 nw1229 vdd vdd pch w=2u l=180n
M10186 t3861 t3859 vdd vdd pch w=2u l=180n
CT3864 t3864 0 0.1f
M10187 t3861 nw1229 t3864 0 nch w=1u l=180n
M10188 t3864 t3859 0 0 nch w=1u l=180n
M10189 nw1231 t3860 vdd vdd pch w=2u l=180n
M10190 nw1231 t3861 vdd vdd pch w=2u l=180n
CT3865 t3865 0 0.1f
M10191 nw1231 t3860 t3865 0 nch w=1u l=180n
M10192 t3865 t3861 0 0 nch w=1u l=180n
Cnw1231 nw1231 0 2f
M10193 nw1232 nw220 vdd vdd pch w=2u l=180n
M10194 nw1232 nw1159 vdd vdd pch w=2u l=180n
CT3866 t3866 0 0.1f
M10195 nw1232 nw220 t3866 0 nch w=1u l=180n
M10196 t3866 nw1159 0 0 nch w=1u l=180n
Cnw1232 nw1232 0 2f
M10197 nw1233 nw1230 vdd vdd pch w=2u l=180n
M10198 nw1233 nw1229 vdd vdd pch w=2u l=180n
CT3867 t3867 0 0.1f
M10199 nw1233 nw1230 t3867 0 nch w=1u l=180n
M10200 t3867 nw1229 0 0 nch w=1u l=180n
Cnw1233 nw1233 0 2f
M10201 nw1234 nw1232 vdd vdd pch w=2u l=180n
M10202 nw1234 nw1233 vdd vdd pch w=2u l=180n
CT3868 t3868 0 0.1f
M10203 nw1234 nw1232 t3868 0 nch w=1u l=180n
M10204 t3868 nw1233 0 0 nch w=1u l=180n
Cnw1234 nw1234 0 2f
CT3869 t3869 0 0.1f
CT3870 t3870 0 0.1f
CT3871 t3871 0 0.1f
M10205 t3869 nw221 vdd vdd pch w=2u l=180n
M10206 t3869 nw1164 vdd vdd pch w=2u l=180n
CT3872 t3872 0 0.1f
M10207 t3869 nw221 t3872 0 nch w=1u l=180n
M10208 t3872 nw1164 0 0 nch w=1u l=180n
M10209 t3870 nw221 vdd vdd pch w=2u l=180n
M10210 t3870 t3869 vdd vdd pch w=2u l=180n
CT3873 t3873 0 0.1f
M10211 t3870 nw221 t3873 0 nch w=1u l=180n
M10212 t3873 t3869 0 0 nch w=1u l=180n
M10213 t3871 nw1164 vdd vdd pch w=2u l=180n
M10214 t3871 t3869 vdd vdd pch w=2u l=180n
CT3874 t3874 0 0.1f
M10215 t3871 nw1164 t3874 0 nch w=1u l=180n
M10216 t3874 t3869 0 0 nch w=1u l=180n
M10217 nw1235 t3870 vdd vdd pch w=2u l=180n
M10218 nw1235 t3871 vdd vdd pch w=2u l=180n
CT3875 t3875 0 0.1f
M10219 nw1235 t3870 t3875 0 nch w=1u l=180n
M10220 t3875 t3871 0 0 nch w=1u l=180n
Cnw1235 nw1235 0 2f
CT3876 t3876 0 0.1f
CT3877 t3877 0 0.1f
CT3878 t3878 0 0.1f
M10221 t3876 nw1235 vdd vdd pch w=2u l=180n
M10222 t3876 nw1234 vdd vdd pch w=2u l=180n
CT3879 t3879 0 0.1f
M10223 t3876 nw1235 t3879 0 nch w=1u l=180n
M10224 t3879 nw1234 0 0 nch w=1u l=180n
M10225 t3877 nw1235 vdd vdd pch w=2u l=180n
M10226 t3877 t3876 vdd vdd pch w=2u l=180n
CT3880 t3880 0 0.1f
M10227 t3877 nw1235 t3880 0 nch w=1u l=180n
M10228 t3880 t3876 0 0 nch w=1u l=180n
M10229 t3878 nw1234 vdd vdd pch w=2u l=180n
M10230 t3878 t3876 vdd vdd pch w=2u l=180n
CT3881 t3881 0 0.1f
M10231 t3878 nw1234 t3881 0 nch w=1u l=180n
M10232 t3881 t3876 0 0 nch w=1u l=180n
M10233 nw1236 t3877 vdd vdd pch w=2u l=180n
M10234 nw1236 t3878 vdd vdd pch w=2u l=180n
CT3882 t3882 0 0.1f
M10235 nw1236 t3877 t3882 0 nch w=1u l=180n
M10236 t3882 t3878 0 0 nch w=1u l=180n
Cnw1236 nw1236 0 2f
M10237 nw1237 nw221 vdd vdd pch w=2u l=180n
M10238 nw1237 nw1164 vdd vdd pch w=2u l=180n
CT3883 t3883 0 0.1f
M10239 nw1237 nw221 t3883 0 nch w=1u l=180n
M10240 t3883 nw1164 0 0 nch w=1u l=180n
Cnw1237 nw1237 0 2f
M10241 nw1238 nw1235 vdd vdd pch w=2u l=180n
M10242 nw1238 nw1234 vdd vdd pch w=2u l=180n
CT3884 t3884 0 0.1f
M10243 nw1238 nw1235 t3884 0 nch w=1u l=180n
M10244 t3884 nw1234 0 0 nch w=1u l=180n
Cnw1238 nw1238 0 2f
M10245 nw1239 nw1237 vdd vdd pch w=2u l=180n
M10246 nw1239 nw1238 vdd vdd pch w=2u l=180n
CT3885 t3885 0 0.1f
M10247 nw1239 nw1237 t3885 0 nch w=1u l=180n
M10248 t3885 nw1238 0 0 nch w=1u l=180n
Cnw1239 nw1239 0 2f
CT3886 t3886 0 0.1f
CT3887 t3887 0 0.1f
CT3888 t3888 0 0.1f
M10249 t3886 nw222 vdd vdd pch w=2u l=180n
M10250 t3886 nw1169 vdd vdd pch w=2u l=180n
CT3889 t3889 0 0.1f
M10251 t3886 nw222 t3889 0 nch w=1u l=180n
M10252 t3889 nw1169 0 0 nch w=1u l=180n
M10253 t3887 nw222 vdd vdd pch w=2u l=180n
M10254 t3887 t3886 vdd vdd pch w=2u l=180n
CT3890 t3890 0 0.1f
M10255 t3887 nw222 t3890 0 nch w=1u l=180n
M10256 t3890 t3886 0 0 nch w=1u l=180n
M10257 t3888 nw1169 vdd vdd pch w=2u l=180n
M10258 t3888 t3886 vdd vdd pch w=2u l=180n
CT3891 t3891 0 0.1f
M10259 t3888 nw1169 t3891 0 nch w=1u l=180n
M10260 t3891 t3886 0 0 nch w=1u l=180n
M10261 nw1240 t3887 vdd vdd pch w=2u l=180n
M10262 nw1240 t3888 vdd vdd pch w=2u l=180n
CT3892 t3892 0 0.1f
M10263 nw1240 t3887 t3892 0 nch w=1u l=180n
M10264 t3892 t3888 0 0 nch w=1u l=180n
Cnw1240 nw1240 0 2f
CT3893 t3893 0 0.1f
CT3894 t3894 0 0.1f
CT3895 t3895 0 0.1f
M10265 t3893 nw1240 vdd vdd pch w=2u l=180n
M10266 t3893 nw1239 vdd vdd pch w=2u l=180n
CT3896 t3896 0 0.1f
M10267 t3893 nw1240 t3896 0 nch w=1u l=180n
M10268 t3896 nw1239 0 0 nch w=1u l=180n
M10269 t3894 nw1240 vdd vdd pch w=2u l=180n
M10270 t3894 t3893 vdd vdd pch w=2u l=180n
CT3897 t3897 0 0.1f
M10271 t3894 nw1240 t3897 0 nch w=1u l=180n
M10272 t3897 t3893 0 0 nch w=1u l=180n
M10273 t3895 nw1239 vdd vdd pch w=2u l=180n
M10274 t3895 t3893 vdd vdd pch w=2u l=180n
CT3898 t3898 0 0.1f
M10275 t3895 nw1239 t3898 0 nch w=1u l=180n
M10276 t3898 t3893 0 0 nch w=1u l=180n
M10277 nw1241 t3894 vdd vdd pch w=2u l=180n
M10278 nw1241 t3895 vdd vdd pch w=2u l=180n
CT3899 t3899 0 0.1f
M10279 nw1241 t3894 t3899 0 nch w=1u l=180n
M10280 t3899 t3895 0 0 nch w=1u l=180n
Cnw1241 nw1241 0 2f
M10281 nw1242 nw222 vdd vdd pch w=2u l=180n
M10282 nw1242 nw1169 vdd vdd pch w=2u l=180n
CT3900 t3900 0 0.1f
M10283 nw1242 nw222 t3900 0 nch w=1u l=180n
M10284 t3900 nw1169 0 0 nch w=1u l=180n
Cnw1242 nw1242 0 2f
M10285 nw1243 nw1240 vdd vdd pch w=2u l=180n
M10286 nw1243 nw1239 vdd vdd pch w=2u l=180n
CT3901 t3901 0 0.1f
M10287 nw1243 nw1240 t3901 0 nch w=1u l=180n
M10288 t3901 nw1239 0 0 nch w=1u l=180n
Cnw1243 nw1243 0 2f
M10289 nw1244 nw1242 vdd vdd pch w=2u l=180n
M10290 nw1244 nw1243 vdd vdd pch w=2u l=180n
CT3902 t3902 0 0.1f
M10291 nw1244 nw1242 t3902 0 nch w=1u l=180n
M10292 t3902 nw1243 0 0 nch w=1u l=180n
Cnw1244 nw1244 0 2f
CT3903 t3903 0 0.1f
CT3904 t3904 0 0.1f
CT3905 t3905 0 0.1f
M10293 t3903 nw223 vdd vdd pch w=2u l=180n
M10294 t3903 nw1174 vdd vdd pch w=2u l=180n
CT3906 t3906 0 0.1f
M10295 t3903 nw223 t3906 0 nch w=1u l=180n
M10296 t3906 nw1174 0 0 nch w=1u l=180n
M10297 t3904 nw223 vdd vdd pch w=2u l=180n
M10298 t3904 t3903 vdd vdd pch w=2u l=180n
CT3907 t3907 0 0.1f
M10299 t3904 nw223 t3907 0 nch w=1u l=180n
M10300 t3907 t3903 0 0 nch w=1u l=180n
M10301 t3905 nw1174 vdd vdd pch w=2u l=180n
M10302 t3905 t3903 vdd vdd pch w=2u l=180n
CT3908 t3908 0 0.1f
M10303 t3905 nw1174 t3908 0 nch w=1u l=180n
M10304 t3908 t3903 0 0 nch w=1u l=180n
M10305 nw1245 t3904 vdd vdd pch w=2u l=180n
M10306 nw1245 t3905 vdd vdd pch w=2u l=180n
CT3909 t3909 0 0.1f
M10307 nw1245 t3904 t3909 0 nch w=1u l=180n
M10308 t3909 t3905 0 0 nch w=1u l=180n
Cnw1245 nw1245 0 2f
CT3910 t3910 0 0.1f
CT3911 t3911 0 0.1f
CT3912 t3912 0 0.1f
M10309 t3910 nw1245 vdd vdd pch w=2u l=180n
M10310 t3910 nw1244 vdd vdd pch w=2u l=180n
CT3913 t3913 0 0.1f
M10311 t3910 nw1245 t3913 0 nch w=1u l=180n
M10312 t3913 nw1244 0 0 nch w=1u l=180n
M10313 t3911 nw1245 vdd vdd pch w=2u l=180n
M10314 t3911 t3910 vdd vdd pch w=2u l=180n
CT3914 t3914 0 0.1f
M10315 t3911 nw1245 t3914 0 nch w=1u l=180n
M10316 t3914 t3910 0 0 nch w=1u l=180n
M10317 t3912 nw1244 vdd vdd pch w=2u l=180n
M10318 t3912 t3910 vdd vdd pch w=2u l=180n
CT3915 t3915 0 0.1f
M10319 t3912 nw1244 t3915 0 nch w=1u l=180n
M10320 t3915 t3910 0 0 nch w=1u l=180n
M10321 nw1246 t3911 vdd vdd pch w=2u l=180n
M10322 nw1246 t3912 vdd vdd pch w=2u l=180n
CT3916 t3916 0 0.1f
M10323 nw1246 t3911 t3916 0 nch w=1u l=180n
M10324 t3916 t3912 0 0 nch w=1u l=180n
Cnw1246 nw1246 0 2f
M10325 nw1247 nw223 vdd vdd pch w=2u l=180n
M10326 nw1247 nw1174 vdd vdd pch w=2u l=180n
CT3917 t3917 0 0.1f
M10327 nw1247 nw223 t3917 0 nch w=1u l=180n
M10328 t3917 nw1174 0 0 nch w=1u l=180n
Cnw1247 nw1247 0 2f
M10329 nw1248 nw1245 vdd vdd pch w=2u l=180n
M10330 nw1248 nw1244 vdd vdd pch w=2u l=180n
CT3918 t3918 0 0.1f
M10331 nw1248 nw1245 t3918 0 nch w=1u l=180n
M10332 t3918 nw1244 0 0 nch w=1u l=180n
Cnw1248 nw1248 0 2f
M10333 nw1249 nw1247 vdd vdd pch w=2u l=180n
M10334 nw1249 nw1248 vdd vdd pch w=2u l=180n
CT3919 t3919 0 0.1f
M10335 nw1249 nw1247 t3919 0 nch w=1u l=180n
M10336 t3919 nw1248 0 0 nch w=1u l=180n
Cnw1249 nw1249 0 2f
CT3920 t3920 0 0.1f
CT3921 t3921 0 0.1f
CT3922 t3922 0 0.1f
M10337 t3920 nw224 vdd vdd pch w=2u l=180n
M10338 t3920 nw1177 vdd vdd pch w=2u l=180n
CT3923 t3923 0 0.1f
M10339 t3920 nw224 t3923 0 nch w=1u l=180n
M10340 t3923 nw1177 0 0 nch w=1u l=180n
M10341 t3921 nw224 vdd vdd pch w=2u l=180n
M10342 t3921 t3920 vdd vdd pch w=2u l=180n
CT3924 t3924 0 0.1f
M10343 t3921 nw224 t3924 0 nch w=1u l=180n
M10344 t3924 t3920 0 0 nch w=1u l=180n
M10345 t3922 nw1177 vdd vdd pch w=2u l=180n
M10346 t3922 t3920 vdd vdd pch w=2u l=180n
CT3925 t3925 0 0.1f
M10347 t3922 nw1177 t3925 0 nch w=1u l=180n
M10348 t3925 t3920 0 0 nch w=1u l=180n
M10349 nw1250 t3921 vdd vdd pch w=2u l=180n
M10350 nw1250 t3922 vdd vdd pch w=2u l=180n
CT3926 t3926 0 0.1f
M10351 nw1250 t3921 t3926 0 nch w=1u l=180n
M10352 t3926 t3922 0 0 nch w=1u l=180n
Cnw1250 nw1250 0 2f
CT3927 t3927 0 0.1f
CT3928 t3928 0 0.1f
CT3929 t3929 0 0.1f
M10353 t3927 nw1250 vdd vdd pch w=2u l=180n
M10354 t3927 nw1249 vdd vdd pch w=2u l=180n
CT3930 t3930 0 0.1f
M10355 t3927 nw1250 t3930 0 nch w=1u l=180n
M10356 t3930 nw1249 0 0 nch w=1u l=180n
M10357 t3928 nw1250 vdd vdd pch w=2u l=180n
M10358 t3928 t3927 vdd vdd pch w=2u l=180n
CT3931 t3931 0 0.1f
M10359 t3928 nw1250 t3931 0 nch w=1u l=180n
M10360 t3931 t3927 0 0 nch w=1u l=180n
M10361 t3929 nw1249 vdd vdd pch w=2u l=180n
M10362 t3929 t3927 vdd vdd pch w=2u l=180n
CT3932 t3932 0 0.1f
M10363 t3929 nw1249 t3932 0 nch w=1u l=180n
M10364 t3932 t3927 0 0 nch w=1u l=180n
M10365 nw1251 t3928 vdd vdd pch w=2u l=180n
M10366 nw1251 t3929 vdd vdd pch w=2u l=180n
CT3933 t3933 0 0.1f
M10367 nw1251 t3928 t3933 0 nch w=1u l=180n
M10368 t3933 t3929 0 0 nch w=1u l=180n
Cnw1251 nw1251 0 2f
M10369 nw1252 nw224 vdd vdd pch w=2u l=180n
M10370 nw1252 nw1177 vdd vdd pch w=2u l=180n
CT3934 t3934 0 0.1f
M10371 nw1252 nw224 t3934 0 nch w=1u l=180n
M10372 t3934 nw1177 0 0 nch w=1u l=180n
Cnw1252 nw1252 0 2f
M10373 nw1253 nw1250 vdd vdd pch w=2u l=180n
M10374 nw1253 nw1249 vdd vdd pch w=2u l=180n
CT3935 t3935 0 0.1f
M10375 nw1253 nw1250 t3935 0 nch w=1u l=180n
M10376 t3935 nw1249 0 0 nch w=1u l=180n
Cnw1253 nw1253 0 2f
M10377 nw1254 nw1252 vdd vdd pch w=2u l=180n
M10378 nw1254 nw1253 vdd vdd pch w=2u l=180n
CT3936 t3936 0 0.1f
M10379 nw1254 nw1252 t3936 0 nch w=1u l=180n
M10380 t3936 nw1253 0 0 nch w=1u l=180n
Cnw1254 nw1254 0 2f
CT3937 t3937 0 0.1f
CT3938 t3938 0 0.1f
CT3939 t3939 0 0.1f
M10381 t3937 nw225 vdd vdd pch w=2u l=180n
M10382 t3937 nw1181 vdd vdd pch w=2u l=180n
CT3940 t3940 0 0.1f
M10383 t3937 nw225 t3940 0 nch w=1u l=180n
M10384 t3940 nw1181 0 0 nch w=1u l=180n
M10385 t3938 nw225 vdd vdd pch w=2u l=180n
M10386 t3938 t3937 vdd vdd pch w=2u l=180n
CT3941 t3941 0 0.1f
M10387 t3938 nw225 t3941 0 nch w=1u l=180n
M10388 t3941 t3937 0 0 nch w=1u l=180n
M10389 t3939 nw1181 vdd vdd pch w=2u l=180n
M10390 t3939 t3937 vdd vdd pch w=2u l=180n
CT3942 t3942 0 0.1f
M10391 t3939 nw1181 t3942 0 nch w=1u l=180n
M10392 t3942 t3937 0 0 nch w=1u l=180n
M10393 nw1255 t3938 vdd vdd pch w=2u l=180n
M10394 nw1255 t3939 vdd vdd pch w=2u l=180n
CT3943 t3943 0 0.1f
M10395 nw1255 t3938 t3943 0 nch w=1u l=180n
M10396 t3943 t3939 0 0 nch w=1u l=180n
Cnw1255 nw1255 0 2f
CT3944 t3944 0 0.1f
M10397 t3944 nw225 vdd vdd pch w=2u l=180n
M10398 t3944 nw1181 vdd vdd pch w=2u l=180n
CT3945 t3945 0 0.1f
M10399 t3944 nw225 t3945 0 nch w=1u l=180n
M10400 t3945 nw1181 0 0 nch w=1u l=180n
M10401 nw1256 t3944 vdd vdd pch w=2u l=180n
M10402 nw1256 t3944 0 0 nch w=1u l=180n
Cnw1256 nw1256 0 2f
CT3946 t3946 0 0.1f
CT3947 t3947 0 0.1f
CT3948 t3948 0 0.1f
M10403 t3946 nw226 vdd vdd pch w=2u l=180n
M10404 t3946 nw1186 vdd vdd pch w=2u l=180n
CT3949 t3949 0 0.1f
M10405 t3946 nw226 t3949 0 nch w=1u l=180n
M10406 t3949 nw1186 0 0 nch w=1u l=180n
M10407 t3947 nw226 vdd vdd pch w=2u l=180n
M10408 t3947 t3946 vdd vdd pch w=2u l=180n
CT3950 t3950 0 0.1f
M10409 t3947 nw226 t3950 0 nch w=1u l=180n
M10410 t3950 t3946 0 0 nch w=1u l=180n
M10411 t3948 nw1186 vdd vdd pch w=2u l=180n
M10412 t3948 t3946 vdd vdd pch w=2u l=180n
CT3951 t3951 0 0.1f
M10413 t3948 nw1186 t3951 0 nch w=1u l=180n
M10414 t3951 t3946 0 0 nch w=1u l=180n
M10415 nw1257 t3947 vdd vdd pch w=2u l=180n
M10416 nw1257 t3948 vdd vdd pch w=2u l=180n
CT3952 t3952 0 0.1f
M10417 nw1257 t3947 t3952 0 nch w=1u l=180n
M10418 t3952 t3948 0 0 nch w=1u l=180n
Cnw1257 nw1257 0 2f
CT3953 t3953 0 0.1f
CT3954 t3954 0 0.1f
CT3955 t3955 0 0.1f
M10419 t3953 nw1257 vdd vdd pch w=2u l=180n
M10420 t3953 nw1256 vdd vdd pch w=2u l=180n
CT3956 t3956 0 0.1f
M10421 t3953 nw1257 t3956 0 nch w=1u l=180n
M10422 t3956 nw1256 0 0 nch w=1u l=180n
M10423 t3954 nw1257 vdd vdd pch w=2u l=180n
M10424 t3954 t3953 vdd vdd pch w=2u l=180n
CT3957 t3957 0 0.1f
M10425 t3954 nw1257 t3957 0 nch w=1u l=180n
M10426 t3957 t3953 0 0 nch w=1u l=180n
M10427 t3955 nw1256 vdd vdd pch w=2u l=180n
M10428 t3955 t3953 vdd vdd pch w=2u l=180n
CT3958 t3958 0 0.1f
M10429 t3955 nw1256 t3958 0 nch w=1u l=180n
M10430 t3958 t3953 0 0 nch w=1u l=180n
M10431 nw1258 t3954 vdd vdd pch w=2u l=180n
M10432 nw1258 t3955 vdd vdd pch w=2u l=180n
CT3959 t3959 0 0.1f
M10433 nw1258 t3954 t3959 0 nch w=1u l=180n
M10434 t3959 t3955 0 0 nch w=1u l=180n
Cnw1258 nw1258 0 2f
M10435 nw1259 nw226 vdd vdd pch w=2u l=180n
M10436 nw1259 nw1186 vdd vdd pch w=2u l=180n
CT3960 t3960 0 0.1f
M10437 nw1259 nw226 t3960 0 nch w=1u l=180n
M10438 t3960 nw1186 0 0 nch w=1u l=180n
Cnw1259 nw1259 0 2f
M10439 nw1260 nw1257 vdd vdd pch w=2u l=180n
M10440 nw1260 nw1256 vdd vdd pch w=2u l=180n
CT3961 t3961 0 0.1f
M10441 nw1260 nw1257 t3961 0 nch w=1u l=180n
M10442 t3961 nw1256 0 0 nch w=1u l=180n
Cnw1260 nw1260 0 2f
M10443 nw1261 nw1259 vdd vdd pch w=2u l=180n
M10444 nw1261 nw1260 vdd vdd pch w=2u l=180n
CT3962 t3962 0 0.1f
M10445 nw1261 nw1259 t3962 0 nch w=1u l=180n
M10446 t3962 nw1260 0 0 nch w=1u l=180n
Cnw1261 nw1261 0 2f
CT3963 t3963 0 0.1f
CT3964 t3964 0 0.1f
CT3965 t3965 0 0.1f
M10447 t3963 nw227 vdd vdd pch w=2u l=180n
M10448 t3963 nw1191 vdd vdd pch w=2u l=180n
CT3966 t3966 0 0.1f
M10449 t3963 nw227 t3966 0 nch w=1u l=180n
M10450 t3966 nw1191 0 0 nch w=1u l=180n
M10451 t3964 nw227 vdd vdd pch w=2u l=180n
M10452 t3964 t3963 vdd vdd pch w=2u l=180n
CT3967 t3967 0 0.1f
M10453 t3964 nw227 t3967 0 nch w=1u l=180n
M10454 t3967 t3963 0 0 nch w=1u l=180n
M10455 t3965 nw1191 vdd vdd pch w=2u l=180n
M10456 t3965 t3963 vdd vdd pch w=2u l=180n
CT3968 t3968 0 0.1f
M10457 t3965 nw1191 t3968 0 nch w=1u l=180n
M10458 t3968 t3963 0 0 nch w=1u l=180n
M10459 nw1262 t3964 vdd vdd pch w=2u l=180n
M10460 nw1262 t3965 vdd vdd pch w=2u l=180n
CT3969 t3969 0 0.1f
M10461 nw1262 t3964 t3969 0 nch w=1u l=180n
M10462 t3969 t3965 0 0 nch w=1u l=180n
Cnw1262 nw1262 0 2f
CT3970 t3970 0 0.1f
CT3971 t3971 0 0.1f
CT3972 t3972 0 0.1f
M10463 t3970 nw1262 vdd vdd pch w=2u l=180n
M10464 t3970 nw1261 vdd vdd pch w=2u l=180n
CT3973 t3973 0 0.1f
M10465 t3970 nw1262 t3973 0 nch w=1u l=180n
M10466 t3973 nw1261 0 0 nch w=1u l=180n
M10467 t3971 nw1262 vdd vdd pch w=2u l=180n
M10468 t3971 t3970 vdd vdd pch w=2u l=180n
CT3974 t3974 0 0.1f
M10469 t3971 nw1262 t3974 0 nch w=1u l=180n
M10470 t3974 t3970 0 0 nch w=1u l=180n
M10471 t3972 nw1261 vdd vdd pch w=2u l=180n
M10472 t3972 t3970 vdd vdd pch w=2u l=180n
CT3975 t3975 0 0.1f
M10473 t3972 nw1261 t3975 0 nch w=1u l=180n
M10474 t3975 t3970 0 0 nch w=1u l=180n
M10475 nw1263 t3971 vdd vdd pch w=2u l=180n
M10476 nw1263 t3972 vdd vdd pch w=2u l=180n
CT3976 t3976 0 0.1f
M10477 nw1263 t3971 t3976 0 nch w=1u l=180n
M10478 t3976 t3972 0 0 nch w=1u l=180n
Cnw1263 nw1263 0 2f
M10479 nw1264 nw227 vdd vdd pch w=2u l=180n
M10480 nw1264 nw1191 vdd vdd pch w=2u l=180n
CT3977 t3977 0 0.1f
M10481 nw1264 nw227 t3977 0 nch w=1u l=180n
M10482 t3977 nw1191 0 0 nch w=1u l=180n
Cnw1264 nw1264 0 2f
M10483 nw1265 nw1262 vdd vdd pch w=2u l=180n
M10484 nw1265 nw1261 vdd vdd pch w=2u l=180n
CT3978 t3978 0 0.1f
M10485 nw1265 nw1262 t3978 0 nch w=1u l=180n
M10486 t3978 nw1261 0 0 nch w=1u l=180n
Cnw1265 nw1265 0 2f
M10487 nw1266 nw1264 vdd vdd pch w=2u l=180n
M10488 nw1266 nw1265 vdd vdd pch w=2u l=180n
CT3979 t3979 0 0.1f
M10489 nw1266 nw1264 t3979 0 nch w=1u l=180n
M10490 t3979 nw1265 0 0 nch w=1u l=180n
Cnw1266 nw1266 0 2f
CT3980 t3980 0 0.1f
CT3981 t3981 0 0.1f
CT3982 t3982 0 0.1f
M10491 t3980 nw228 vdd vdd pch w=2u l=180n
M10492 t3980 nw1196 vdd vdd pch w=2u l=180n
CT3983 t3983 0 0.1f
M10493 t3980 nw228 t3983 0 nch w=1u l=180n
M10494 t3983 nw1196 0 0 nch w=1u l=180n
M10495 t3981 nw228 vdd vdd pch w=2u l=180n
M10496 t3981 t3980 vdd vdd pch w=2u l=180n
CT3984 t3984 0 0.1f
M10497 t3981 nw228 t3984 0 nch w=1u l=180n
M10498 t3984 t3980 0 0 nch w=1u l=180n
M10499 t3982 nw1196 vdd vdd pch w=2u l=180n
M10500 t3982 t3980 vdd vdd pch w=2u l=180n
CT3985 t3985 0 0.1f
M10501 t3982 nw1196 t3985 0 nch w=1u l=180n
M10502 t3985 t3980 0 0 nch w=1u l=180n
M10503 nw1267 t3981 vdd vdd pch w=2u l=180n
M10504 nw1267 t3982 vdd vdd pch w=2u l=180n
CT3986 t3986 0 0.1f
M10505 nw1267 t3981 t3986 0 nch w=1u l=180n
M10506 t3986 t3982 0 0 nch w=1u l=180n
Cnw1267 nw1267 0 2f
CT3987 t3987 0 0.1f
CT3988 t3988 0 0.1f
CT3989 t3989 0 0.1f
M10507 t3987 nw1267 vdd vdd pch w=2u l=180n
M10508 t3987 nw1266 vdd vdd pch w=2u l=180n
CT3990 t3990 0 0.1f
M10509 t3987 nw1267 t3990 0 nch w=1u l=180n
M10510 t3990 nw1266 0 0 nch w=1u l=180n
M10511 t3988 nw1267 vdd vdd pch w=2u l=180n
M10512 t3988 t3987 vdd vdd pch w=2u l=180n
CT3991 t3991 0 0.1f
M10513 t3988 nw1267 t3991 0 nch w=1u l=180n
M10514 t3991 t3987 0 0 nch w=1u l=180n
M10515 t3989 nw1266 vdd vdd pch w=2u l=180n
M10516 t3989 t3987 vdd vdd pch w=2u l=180n
CT3992 t3992 0 0.1f
M10517 t3989 nw1266 t3992 0 nch w=1u l=180n
M10518 t3992 t3987 0 0 nch w=1u l=180n
M10519 nw1268 t3988 vdd vdd pch w=2u l=180n
M10520 nw1268 t3989 vdd vdd pch w=2u l=180n
CT3993 t3993 0 0.1f
M10521 nw1268 t3988 t3993 0 nch w=1u l=180n
M10522 t3993 t3989 0 0 nch w=1u l=180n
Cnw1268 nw1268 0 2f
M10523 nw1269 nw228 vdd vdd pch w=2u l=180n
M10524 nw1269 nw1196 vdd vdd pch w=2u l=180n
CT3994 t3994 0 0.1f
M10525 nw1269 nw228 t3994 0 nch w=1u l=180n
M10526 t3994 nw1196 0 0 nch w=1u l=180n
Cnw1269 nw1269 0 2f
M10527 nw1270 nw1267 vdd vdd pch w=2u l=180n
M10528 nw1270 nw1266 vdd vdd pch w=2u l=180n
CT3995 t3995 0 0.1f
M10529 nw1270 nw1267 t3995 0 nch w=1u l=180n
M10530 t3995 nw1266 0 0 nch w=1u l=180n
Cnw1270 nw1270 0 2f
M10531 nw1271 nw1269 vdd vdd pch w=2u l=180n
M10532 nw1271 nw1270 vdd vdd pch w=2u l=180n
CT3996 t3996 0 0.1f
M10533 nw1271 nw1269 t3996 0 nch w=1u l=180n
M10534 t3996 nw1270 0 0 nch w=1u l=180n
Cnw1271 nw1271 0 2f
CT3997 t3997 0 0.1f
CT3998 t3998 0 0.1f
CT3999 t3999 0 0.1f
M10535 t3997 nw229 vdd vdd pch w=2u l=180n
M10536 t3997 nw1201 vdd vdd pch w=2u l=180n
CT4000 t4000 0 0.1f
M10537 t3997 nw229 t4000 0 nch w=1u l=180n
M10538 t4000 nw1201 0 0 nch w=1u l=180n
M10539 t3998 nw229 vdd vdd pch w=2u l=180n
M10540 t3998 t3997 vdd vdd pch w=2u l=180n
CT4001 t4001 0 0.1f
M10541 t3998 nw229 t4001 0 nch w=1u l=180n
M10542 t4001 t3997 0 0 nch w=1u l=180n
M10543 t3999 nw1201 vdd vdd pch w=2u l=180n
M10544 t3999 t3997 vdd vdd pch w=2u l=180n
CT4002 t4002 0 0.1f
M10545 t3999 nw1201 t4002 0 nch w=1u l=180n
M10546 t4002 t3997 0 0 nch w=1u l=180n
M10547 nw1272 t3998 vdd vdd pch w=2u l=180n
M10548 nw1272 t3999 vdd vdd pch w=2u l=180n
CT4003 t4003 0 0.1f
M10549 nw1272 t3998 t4003 0 nch w=1u l=180n
M10550 t4003 t3999 0 0 nch w=1u l=180n
Cnw1272 nw1272 0 2f
CT4004 t4004 0 0.1f
CT4005 t4005 0 0.1f
CT4006 t4006 0 0.1f
M10551 t4004 nw1272 vdd vdd pch w=2u l=180n
M10552 t4004 nw1271 vdd vdd pch w=2u l=180n
CT4007 t4007 0 0.1f
M10553 t4004 nw1272 t4007 0 nch w=1u l=180n
M10554 t4007 nw1271 0 0 nch w=1u l=180n
M10555 t4005 nw1272 vdd vdd pch w=2u l=180n
M10556 t4005 t4004 vdd vdd pch w=2u l=180n
CT4008 t4008 0 0.1f
M10557 t4005 nw1272 t4008 0 nch w=1u l=180n
M10558 t4008 t4004 0 0 nch w=1u l=180n
M10559 t4006 nw1271 vdd vdd pch w=2u l=180n
M10560 t4006 t4004 vdd vdd pch w=2u l=180n
CT4009 t4009 0 0.1f
M10561 t4006 nw1271 t4009 0 nch w=1u l=180n
M10562 t4009 t4004 0 0 nch w=1u l=180n
M10563 nw1273 t4005 vdd vdd pch w=2u l=180n
M10564 nw1273 t4006 vdd vdd pch w=2u l=180n
CT4010 t4010 0 0.1f
M10565 nw1273 t4005 t4010 0 nch w=1u l=180n
M10566 t4010 t4006 0 0 nch w=1u l=180n
Cnw1273 nw1273 0 2f
M10567 nw1274 nw229 vdd vdd pch w=2u l=180n
M10568 nw1274 nw1201 vdd vdd pch w=2u l=180n
CT4011 t4011 0 0.1f
M10569 nw1274 nw229 t4011 0 nch w=1u l=180n
M10570 t4011 nw1201 0 0 nch w=1u l=180n
Cnw1274 nw1274 0 2f
M10571 nw1275 nw1272 vdd vdd pch w=2u l=180n
M10572 nw1275 nw1271 vdd vdd pch w=2u l=180n
CT4012 t4012 0 0.1f
M10573 nw1275 nw1272 t4012 0 nch w=1u l=180n
M10574 t4012 nw1271 0 0 nch w=1u l=180n
Cnw1275 nw1275 0 2f
M10575 nw1276 nw1274 vdd vdd pch w=2u l=180n
M10576 nw1276 nw1275 vdd vdd pch w=2u l=180n
CT4013 t4013 0 0.1f
M10577 nw1276 nw1274 t4013 0 nch w=1u l=180n
M10578 t4013 nw1275 0 0 nch w=1u l=180n
Cnw1276 nw1276 0 2f
CT4014 t4014 0 0.1f
CT4015 t4015 0 0.1f
CT4016 t4016 0 0.1f
M10579 t4014 nw230 vdd vdd pch w=2u l=180n
M10580 t4014 nw1206 vdd vdd pch w=2u l=180n
CT4017 t4017 0 0.1f
M10581 t4014 nw230 t4017 0 nch w=1u l=180n
M10582 t4017 nw1206 0 0 nch w=1u l=180n
M10583 t4015 nw230 vdd vdd pch w=2u l=180n
M10584 t4015 t4014 vdd vdd pch w=2u l=180n
CT4018 t4018 0 0.1f
M10585 t4015 nw230 t4018 0 nch w=1u l=180n
M10586 t4018 t4014 0 0 nch w=1u l=180n
M10587 t4016 nw1206 vdd vdd pch w=2u l=180n
M10588 t4016 t4014 vdd vdd pch w=2u l=180n
CT4019 t4019 0 0.1f
M10589 t4016 nw1206 t4019 0 nch w=1u l=180n
M10590 t4019 t4014 0 0 nch w=1u l=180n
M10591 nw1277 t4015 vdd vdd pch w=2u l=180n
M10592 nw1277 t4016 vdd vdd pch w=2u l=180n
CT4020 t4020 0 0.1f
M10593 nw1277 t4015 t4020 0 nch w=1u l=180n
M10594 t4020 t4016 0 0 nch w=1u l=180n
Cnw1277 nw1277 0 2f
CT4021 t4021 0 0.1f
CT4022 t4022 0 0.1f
CT4023 t4023 0 0.1f
M10595 t4021 nw1277 vdd vdd pch w=2u l=180n
M10596 t4021 nw1276 vdd vdd pch w=2u l=180n
CT4024 t4024 0 0.1f
M10597 t4021 nw1277 t4024 0 nch w=1u l=180n
M10598 t4024 nw1276 0 0 nch w=1u l=180n
M10599 t4022 nw1277 vdd vdd pch w=2u l=180n
M10600 t4022 t4021 vdd vdd pch w=2u l=180n
CT4025 t4025 0 0.1f
M10601 t4022 nw1277 t4025 0 nch w=1u l=180n
M10602 t4025 t4021 0 0 nch w=1u l=180n
M10603 t4023 nw1276 vdd vdd pch w=2u l=180n
M10604 t4023 t4021 vdd vdd pch w=2u l=180n
CT4026 t4026 0 0.1f
M10605 t4023 nw1276 t4026 0 nch w=1u l=180n
M10606 t4026 t4021 0 0 nch w=1u l=180n
M10607 nw1278 t4022 vdd vdd pch w=2u l=180n
M10608 nw1278 t4023 vdd vdd pch w=2u l=180n
CT4027 t4027 0 0.1f
M10609 nw1278 t4022 t4027 0 nch w=1u l=180n
M10610 t4027 t4023 0 0 nch w=1u l=180n
Cnw1278 nw1278 0 2f
M10611 nw1279 nw230 vdd vdd pch w=2u l=180n
M10612 nw1279 nw1206 vdd vdd pch w=2u l=180n
CT4028 t4028 0 0.1f
M10613 nw1279 nw230 t4028 0 nch w=1u l=180n
M10614 t4028 nw1206 0 0 nch w=1u l=180n
Cnw1279 nw1279 0 2f
M10615 nw1280 nw1277 vdd vdd pch w=2u l=180n
M10616 nw1280 nw1276 vdd vdd pch w=2u l=180n
CT4029 t4029 0 0.1f
M10617 nw1280 nw1277 t4029 0 nch w=1u l=180n
M10618 t4029 nw1276 0 0 nch w=1u l=180n
Cnw1280 nw1280 0 2f
M10619 nw1281 nw1279 vdd vdd pch w=2u l=180n
M10620 nw1281 nw1280 vdd vdd pch w=2u l=180n
CT4030 t4030 0 0.1f
M10621 nw1281 nw1279 t4030 0 nch w=1u l=180n
M10622 t4030 nw1280 0 0 nch w=1u l=180n
Cnw1281 nw1281 0 2f
CT4031 t4031 0 0.1f
CT4032 t4032 0 0.1f
CT4033 t4033 0 0.1f
M10623 t4031 nw231 vdd vdd pch w=2u l=180n
M10624 t4031 nw1211 vdd vdd pch w=2u l=180n
CT4034 t4034 0 0.1f
M10625 t4031 nw231 t4034 0 nch w=1u l=180n
M10626 t4034 nw1211 0 0 nch w=1u l=180n
M10627 t4032 nw231 vdd vdd pch w=2u l=180n
M10628 t4032 t4031 vdd vdd pch w=2u l=180n
CT4035 t4035 0 0.1f
M10629 t4032 nw231 t4035 0 nch w=1u l=180n
M10630 t4035 t4031 0 0 nch w=1u l=180n
M10631 t4033 nw1211 vdd vdd pch w=2u l=180n
M10632 t4033 t4031 vdd vdd pch w=2u l=180n
CT4036 t4036 0 0.1f
M10633 t4033 nw1211 t4036 0 nch w=1u l=180n
M10634 t4036 t4031 0 0 nch w=1u l=180n
M10635 nw1282 t4032 vdd vdd pch w=2u l=180n
M10636 nw1282 t4033 vdd vdd pch w=2u l=180n
CT4037 t4037 0 0.1f
M10637 nw1282 t4032 t4037 0 nch w=1u l=180n
M10638 t4037 t4033 0 0 nch w=1u l=180n
Cnw1282 nw1282 0 2f
CT4038 t4038 0 0.1f
CT4039 t4039 0 0.1f
CT4040 t4040 0 0.1f
M10639 t4038 nw1282 vdd vdd pch w=2u l=180n
M10640 t4038 nw1281 vdd vdd pch w=2u l=180n
CT4041 t4041 0 0.1f
M10641 t4038 nw1282 t4041 0 nch w=1u l=180n
M10642 t4041 nw1281 0 0 nch w=1u l=180n
M10643 t4039 nw1282 vdd vdd pch w=2u l=180n
M10644 t4039 t4038 vdd vdd pch w=2u l=180n
CT4042 t4042 0 0.1f
M10645 t4039 nw1282 t4042 0 nch w=1u l=180n
M10646 t4042 t4038 0 0 nch w=1u l=180n
M10647 t4040 nw1281 vdd vdd pch w=2u l=180n
M10648 t4040 t4038 vdd vdd pch w=2u l=180n
CT4043 t4043 0 0.1f
M10649 t4040 nw1281 t4043 0 nch w=1u l=180n
M10650 t4043 t4038 0 0 nch w=1u l=180n
M10651 nw1283 t4039 vdd vdd pch w=2u l=180n
M10652 nw1283 t4040 vdd vdd pch w=2u l=180n
CT4044 t4044 0 0.1f
M10653 nw1283 t4039 t4044 0 nch w=1u l=180n
M10654 t4044 t4040 0 0 nch w=1u l=180n
Cnw1283 nw1283 0 2f
M10655 nw1284 nw231 vdd vdd pch w=2u l=180n
M10656 nw1284 nw1211 vdd vdd pch w=2u l=180n
CT4045 t4045 0 0.1f
M10657 nw1284 nw231 t4045 0 nch w=1u l=180n
M10658 t4045 nw1211 0 0 nch w=1u l=180n
Cnw1284 nw1284 0 2f
M10659 nw1285 nw1282 vdd vdd pch w=2u l=180n
M10660 nw1285 nw1281 vdd vdd pch w=2u l=180n
CT4046 t4046 0 0.1f
M10661 nw1285 nw1282 t4046 0 nch w=1u l=180n
M10662 t4046 nw1281 0 0 nch w=1u l=180n
Cnw1285 nw1285 0 2f
M10663 nw1286 nw1284 vdd vdd pch w=2u l=180n
M10664 nw1286 nw1285 vdd vdd pch w=2u l=180n
CT4047 t4047 0 0.1f
M10665 nw1286 nw1284 t4047 0 nch w=1u l=180n
M10666 t4047 nw1285 0 0 nch w=1u l=180n
Cnw1286 nw1286 0 2f
CT4048 t4048 0 0.1f
CT4049 t4049 0 0.1f
CT4050 t4050 0 0.1f
M10667 t4048 nw232 vdd vdd pch w=2u l=180n
M10668 t4048 nw1216 vdd vdd pch w=2u l=180n
CT4051 t4051 0 0.1f
M10669 t4048 nw232 t4051 0 nch w=1u l=180n
M10670 t4051 nw1216 0 0 nch w=1u l=180n
M10671 t4049 nw232 vdd vdd pch w=2u l=180n
M10672 t4049 t4048 vdd vdd pch w=2u l=180n
CT4052 t4052 0 0.1f
M10673 t4049 nw232 t4052 0 nch w=1u l=180n
M10674 t4052 t4048 0 0 nch w=1u l=180n
M10675 t4050 nw1216 vdd vdd pch w=2u l=180n
M10676 t4050 t4048 vdd vdd pch w=2u l=180n
CT4053 t4053 0 0.1f
M10677 t4050 nw1216 t4053 0 nch w=1u l=180n
M10678 t4053 t4048 0 0 nch w=1u l=180n
M10679 nw1287 t4049 vdd vdd pch w=2u l=180n
M10680 nw1287 t4050 vdd vdd pch w=2u l=180n
CT4054 t4054 0 0.1f
M10681 nw1287 t4049 t4054 0 nch w=1u l=180n
M10682 t4054 t4050 0 0 nch w=1u l=180n
Cnw1287 nw1287 0 2f
CT4055 t4055 0 0.1f
CT4056 t4056 0 0.1f
CT4057 t4057 0 0.1f
M10683 t4055 nw1287 vdd vdd pch w=2u l=180n
M10684 t4055 nw1286 vdd vdd pch w=2u l=180n
CT4058 t4058 0 0.1f
M10685 t4055 nw1287 t4058 0 nch w=1u l=180n
M10686 t4058 nw1286 0 0 nch w=1u l=180n
M10687 t4056 nw1287 vdd vdd pch w=2u l=180n
M10688 t4056 t4055 vdd vdd pch w=2u l=180n
CT4059 t4059 0 0.1f
M10689 t4056 nw1287 t4059 0 nch w=1u l=180n
M10690 t4059 t4055 0 0 nch w=1u l=180n
M10691 t4057 nw1286 vdd vdd pch w=2u l=180n
M10692 t4057 t4055 vdd vdd pch w=2u l=180n
CT4060 t4060 0 0.1f
M10693 t4057 nw1286 t4060 0 nch w=1u l=180n
M10694 t4060 t4055 0 0 nch w=1u l=180n
M10695 nw1288 t4056 vdd vdd pch w=2u l=180n
M10696 nw1288 t4057 vdd vdd pch w=2u l=180n
CT4061 t4061 0 0.1f
M10697 nw1288 t4056 t4061 0 nch w=1u l=180n
M10698 t4061 t4057 0 0 nch w=1u l=180n
Cnw1288 nw1288 0 2f
M10699 nw1289 nw232 vdd vdd pch w=2u l=180n
M10700 nw1289 nw1216 vdd vdd pch w=2u l=180n
CT4062 t4062 0 0.1f
M10701 nw1289 nw232 t4062 0 nch w=1u l=180n
M10702 t4062 nw1216 0 0 nch w=1u l=180n
Cnw1289 nw1289 0 2f
M10703 nw1290 nw1287 vdd vdd pch w=2u l=180n
M10704 nw1290 nw1286 vdd vdd pch w=2u l=180n
CT4063 t4063 0 0.1f
M10705 nw1290 nw1287 t4063 0 nch w=1u l=180n
M10706 t4063 nw1286 0 0 nch w=1u l=180n
Cnw1290 nw1290 0 2f
M10707 nw1291 nw1289 vdd vdd pch w=2u l=180n
M10708 nw1291 nw1290 vdd vdd pch w=2u l=180n
CT4064 t4064 0 0.1f
M10709 nw1291 nw1289 t4064 0 nch w=1u l=180n
M10710 t4064 nw1290 0 0 nch w=1u l=180n
Cnw1291 nw1291 0 2f
CT4065 t4065 0 0.1f
CT4066 t4066 0 0.1f
CT4067 t4067 0 0.1f
M10711 t4065 nw233 vdd vdd pch w=2u l=180n
M10712 t4065 nw1221 vdd vdd pch w=2u l=180n
CT4068 t4068 0 0.1f
M10713 t4065 nw233 t4068 0 nch w=1u l=180n
M10714 t4068 nw1221 0 0 nch w=1u l=180n
M10715 t4066 nw233 vdd vdd pch w=2u l=180n
M10716 t4066 t4065 vdd vdd pch w=2u l=180n
CT4069 t4069 0 0.1f
M10717 t4066 nw233 t4069 0 nch w=1u l=180n
M10718 t4069 t4065 0 0 nch w=1u l=180n
M10719 t4067 nw1221 vdd vdd pch w=2u l=180n
M10720 t4067 t4065 vdd vdd pch w=2u l=180n
CT4070 t4070 0 0.1f
M10721 t4067 nw1221 t4070 0 nch w=1u l=180n
M10722 t4070 t4065 0 0 nch w=1u l=180n
M10723 nw1292 t4066 vdd vdd pch w=2u l=180n
M10724 nw1292 t4067 vdd vdd pch w=2u l=180n
CT4071 t4071 0 0.1f
M10725 nw1292 t4066 t4071 0 nch w=1u l=180n
M10726 t4071 t4067 0 0 nch w=1u l=180n
Cnw1292 nw1292 0 2f
CT4072 t4072 0 0.1f
CT4073 t4073 0 0.1f
CT4074 t4074 0 0.1f
M10727 t4072 nw1292 vdd vdd pch w=2u l=180n
M10728 t4072 nw1291 vdd vdd pch w=2u l=180n
CT4075 t4075 0 0.1f
M10729 t4072 nw1292 t4075 0 nch w=1u l=180n
M10730 t4075 nw1291 0 0 nch w=1u l=180n
M10731 t4073 nw1292 vdd vdd pch w=2u l=180n
M10732 t4073 t4072 vdd vdd pch w=2u l=180n
CT4076 t4076 0 0.1f
M10733 t4073 nw1292 t4076 0 nch w=1u l=180n
M10734 t4076 t4072 0 0 nch w=1u l=180n
M10735 t4074 nw1291 vdd vdd pch w=2u l=180n
M10736 t4074 t4072 vdd vdd pch w=2u l=180n
CT4077 t4077 0 0.1f
M10737 t4074 nw1291 t4077 0 nch w=1u l=180n
M10738 t4077 t4072 0 0 nch w=1u l=180n
M10739 nw1293 t4073 vdd vdd pch w=2u l=180n
M10740 nw1293 t4074 vdd vdd pch w=2u l=180n
CT4078 t4078 0 0.1f
M10741 nw1293 t4073 t4078 0 nch w=1u l=180n
M10742 t4078 t4074 0 0 nch w=1u l=180n
Cnw1293 nw1293 0 2f
M10743 nw1294 nw233 vdd vdd pch w=2u l=180n
M10744 nw1294 nw1221 vdd vdd pch w=2u l=180n
CT4079 t4079 0 0.1f
M10745 nw1294 nw233 t4079 0 nch w=1u l=180n
M10746 t4079 nw1221 0 0 nch w=1u l=180n
Cnw1294 nw1294 0 2f
M10747 nw1295 nw1292 vdd vdd pch w=2u l=180n
M10748 nw1295 nw1291 vdd vdd pch w=2u l=180n
CT4080 t4080 0 0.1f
M10749 nw1295 nw1292 t4080 0 nch w=1u l=180n
M10750 t4080 nw1291 0 0 nch w=1u l=180n
Cnw1295 nw1295 0 2f
M10751 nw1296 nw1294 vdd vdd pch w=2u l=180n
M10752 nw1296 nw1295 vdd vdd pch w=2u l=180n
CT4081 t4081 0 0.1f
M10753 nw1296 nw1294 t4081 0 nch w=1u l=180n
M10754 t4081 nw1295 0 0 nch w=1u l=180n
Cnw1296 nw1296 0 2f
CT4082 t4082 0 0.1f
CT4083 t4083 0 0.1f
CT4084 t4084 0 0.1f
M10755 t4082 nw234 vdd vdd pch w=2u l=180n
M10756 t4082 nw1226 vdd vdd pch w=2u l=180n
CT4085 t4085 0 0.1f
M10757 t4082 nw234 t4085 0 nch w=1u l=180n
M10758 t4085 nw1226 0 0 nch w=1u l=180n
M10759 t4083 nw234 vdd vdd pch w=2u l=180n
M10760 t4083 t4082 vdd vdd pch w=2u l=180n
CT4086 t4086 0 0.1f
M10761 t4083 nw234 t4086 0 nch w=1u l=180n
M10762 t4086 t4082 0 0 nch w=1u l=180n
M10763 t4084 nw1226 vdd vdd pch w=2u l=180n
M10764 t4084 t4082 vdd vdd pch w=2u l=180n
CT4087 t4087 0 0.1f
M10765 t4084 nw1226 t4087 0 nch w=1u l=180n
M10766 t4087 t4082 0 0 nch w=1u l=180n
M10767 nw1297 t4083 vdd vdd pch w=2u l=180n
M10768 nw1297 t4084 vdd vdd pch w=2u l=180n
CT4088 t4088 0 0.1f
M10769 nw1297 t4083 t4088 0 nch w=1u l=180n
M10770 t4088 t4084 0 0 nch w=1u l=180n
Cnw1297 nw1297 0 2f
CT4089 t4089 0 0.1f
CT4090 t4090 0 0.1f
CT4091 t4091 0 0.1f
M10771 t4089 nw1297 vdd vdd pch w=2u l=180n
M10772 t4089 nw1296 vdd vdd pch w=2u l=180n
CT4092 t4092 0 0.1f
M10773 t4089 nw1297 t4092 0 nch w=1u l=180n
M10774 t4092 nw1296 0 0 nch w=1u l=180n
M10775 t4090 nw1297 vdd vdd pch w=2u l=180n
M10776 t4090 t4089 vdd vdd pch w=2u l=180n
CT4093 t4093 0 0.1f
M10777 t4090 nw1297 t4093 0 nch w=1u l=180n
M10778 t4093 t4089 0 0 nch w=1u l=180n
M10779 t4091 nw1296 vdd vdd pch w=2u l=180n
M10780 t4091 t4089 vdd vdd pch w=2u l=180n
CT4094 t4094 0 0.1f
M10781 t4091 nw1296 t4094 0 nch w=1u l=180n
M10782 t4094 t4089 0 0 nch w=1u l=180n
M10783 nw1298 t4090 vdd vdd pch w=2u l=180n
M10784 nw1298 t4091 vdd vdd pch w=2u l=180n
CT4095 t4095 0 0.1f
M10785 nw1298 t4090 t4095 0 nch w=1u l=180n
M10786 t4095 t4091 0 0 nch w=1u l=180n
Cnw1298 nw1298 0 2f
M10787 nw1299 nw234 vdd vdd pch w=2u l=180n
M10788 nw1299 nw1226 vdd vdd pch w=2u l=180n
CT4096 t4096 0 0.1f
M10789 nw1299 nw234 t4096 0 nch w=1u l=180n
M10790 t4096 nw1226 0 0 nch w=1u l=180n
Cnw1299 nw1299 0 2f
M10791 nw1300 nw1297 vdd vdd pch w=2u l=180n
M10792 nw1300 nw1296 vdd vdd pch w=2u l=180n
CT4097 t4097 0 0.1f
M10793 nw1300 nw1297 t4097 0 nch w=1u l=180n
M10794 t4097 nw1296 0 0 nch w=1u l=180n
Cnw1300 nw1300 0 2f
M10795 nw1301 nw1299 vdd vdd pch w=2u l=180n
M10796 nw1301 nw1300 vdd vdd pch w=2u l=180n
CT4098 t4098 0 0.1f
M10797 nw1301 nw1299 t4098 0 nch w=1u l=180n
M10798 t4098 nw1300 0 0 nch w=1u l=180n
Cnw1301 nw1301 0 2f
CT4099 t4099 0 0.1f
CT4100 t4100 0 0.1f
CT4101 t4101 0 0.1f
M10799 t4099 nw235 vdd vdd pch w=2u l=180n
M10800 t4099 nw1231 vdd vdd pch w=2u l=180n
CT4102 t4102 0 0.1f
M10801 t4099 nw235 t4102 0 nch w=1u l=180n
M10802 t4102 nw1231 0 0 nch w=1u l=180n
M10803 t4100 nw235 vdd vdd pch w=2u l=180n
M10804 t4100 t4099 vdd vdd pch w=2u l=180n
CT4103 t4103 0 0.1f
M10805 t4100 nw235 t4103 0 nch w=1u l=180n
M10806 t4103 t4099 0 0 nch w=1u l=180n
M10807 t4101 nw1231 vdd vdd pch w=2u l=180n
M10808 t4101 t4099 vdd vdd pch w=2u l=180n
CT4104 t4104 0 0.1f
M10809 t4101 nw1231 t4104 0 nch w=1u l=180n
M10810 t4104 t4099 0 0 nch w=1u l=180n
M10811 nw1302 t4100 vdd vdd pch w=2u l=180n
M10812 nw1302 t4101 vdd vdd pch w=2u l=180n
CT4105 t4105 0 0.1f
M10813 nw1302 t4100 t4105 0 nch w=1u l=180n
M10814 t4105 t4101 0 0 nch w=1u l=180n
Cnw1302 nw1302 0 2f
CT4106 t4106 0 0.1f
CT4107 t4107 0 0.1f
CT4108 t4108 0 0.1f
M10815 t4106 nw1302 vdd vdd pch w=2u l=180n
M10816 t4106 nw1301 vdd vdd pch w=2u l=180n
CT4109 t4109 0 0.1f
M10817 t4106 nw1302 t4109 0 nch w=1u l=180n
M10818 t4109 nw1301 0 0 nch w=1u l=180n
M10819 t4107 nw1302 vdd vdd pch w=2u l=180n
M10820 t4107 t4106 vdd vdd pch w=2u l=180n
CT4110 t4110 0 0.1f
M10821 t4107 nw1302 t4110 0 nch w=1u l=180n
M10822 t4110 t4106 0 0 nch w=1u l=180n
M10823 t4108 nw1301 vdd vdd pch w=2u l=180n
M10824 t4108 t4106 vdd vdd pch w=2u l=180n
CT4111 t4111 0 0.1f
M10825 t4108 nw1301 t4111 0 nch w=1u l=180n
M10826 t4111 t4106 0 0 nch w=1u l=180n
M10827 nw1303 t4107 vdd vdd pch w=2u l=180n
M10828 nw1303 t4108 vdd vdd pch w=2u l=180n
CT4112 t4112 0 0.1f
M10829 nw1303 t4107 t4112 0 nch w=1u l=180n
M10830 t4112 t4108 0 0 nch w=1u l=180n
Cnw1303 nw1303 0 2f
M10831 nw1304 nw235 vdd vdd pch w=2u l=180n
M10832 nw1304 nw1231 vdd vdd pch w=2u l=180n
CT4113 t4113 0 0.1f
M10833 nw1304 nw235 t4113 0 nch w=1u l=180n
M10834 t4113 nw1231 0 0 nch w=1u l=180n
Cnw1304 nw1304 0 2f
M10835 nw1305 nw1302 vdd vdd pch w=2u l=180n
M10836 nw1305 nw1301 vdd vdd pch w=2u l=180n
CT4114 t4114 0 0.1f
M10837 nw1305 nw1302 t4114 0 nch w=1u l=180n
M10838 t4114 nw1301 0 0 nch w=1u l=180n
Cnw1305 nw1305 0 2f
M10839 nw1306 nw1304 vdd vdd pch w=2u l=180n
M10840 nw1306 nw1305 vdd vdd pch w=2u l=180n
CT4115 t4115 0 0.1f
M10841 nw1306 nw1304 t4115 0 nch w=1u l=180n
M10842 t4115 nw1305 0 0 nch w=1u l=180n
Cnw1306 nw1306 0 2f
CT4116 t4116 0 0.1f
CT4117 t4117 0 0.1f
CT4118 t4118 0 0.1f
M10843 t4116 nw236 vdd vdd pch w=2u l=180n
M10844 t4116 nw1236 vdd vdd pch w=2u l=180n
CT4119 t4119 0 0.1f
M10845 t4116 nw236 t4119 0 nch w=1u l=180n
M10846 t4119 nw1236 0 0 nch w=1u l=180n
M10847 t4117 nw236 vdd vdd pch w=2u l=180n
M10848 t4117 t4116 vdd vdd pch w=2u l=180n
CT4120 t4120 0 0.1f
M10849 t4117 nw236 t4120 0 nch w=1u l=180n
M10850 t4120 t4116 0 0 nch w=1u l=180n
M10851 t4118 nw1236 vdd vdd pch w=2u l=180n
M10852 t4118 t4116 vdd vdd pch w=2u l=180n
CT4121 t4121 0 0.1f
M10853 t4118 nw1236 t4121 0 nch w=1u l=180n
M10854 t4121 t4116 0 0 nch w=1u l=180n
M10855 nw1307 t4117 vdd vdd pch w=2u l=180n
M10856 nw1307 t4118 vdd vdd pch w=2u l=180n
CT4122 t4122 0 0.1f
M10857 nw1307 t4117 t4122 0 nch w=1u l=180n
M10858 t4122 t4118 0 0 nch w=1u l=180n
Cnw1307 nw1307 0 2f
CT4123 t4123 0 0.1f
CT4124 t4124 0 0.1f
CT4125 t4125 0 0.1f
M10859 t4123 nw1307 vdd vdd pch w=2u l=180n
M10860 t4123 nw1306 vdd vdd pch w=2u l=180n
CT4126 t4126 0 0.1f
M10861 t4123 nw1307 t4126 0 nch w=1u l=180n
M10862 t4126 nw1306 0 0 nch w=1u l=180n
M10863 t4124 nw1307 vdd vdd pch w=2u l=180n
M10864 t4124 t4123 vdd vdd pch w=2u l=180n
CT4127 t4127 0 0.1f
M10865 t4124 nw1307 t4127 0 nch w=1u l=180n
M10866 t4127 t4123 0 0 nch w=1u l=180n
M10867 t4125 nw1306 vdd vdd pch w=2u l=180n
M10868 t4125 t4123 vdd vdd pch w=2u l=180n
CT4128 t4128 0 0.1f
M10869 t4125 nw1306 t4128 0 nch w=1u l=180n
M10870 t4128 t4123 0 0 nch w=1u l=180n
M10871 nw1308 t4124 vdd vdd pch w=2u l=180n
M10872 nw1308 t4125 vdd vdd pch w=2u l=180n
CT4129 t4129 0 0.1f
M10873 nw1308 t4124 t4129 0 nch w=1u l=180n
M10874 t4129 t4125 0 0 nch w=1u l=180n
Cnw1308 nw1308 0 2f
M10875 nw1309 nw236 vdd vdd pch w=2u l=180n
M10876 nw1309 nw1236 vdd vdd pch w=2u l=180n
CT4130 t4130 0 0.1f
M10877 nw1309 nw236 t4130 0 nch w=1u l=180n
M10878 t4130 nw1236 0 0 nch w=1u l=180n
Cnw1309 nw1309 0 2f
M10879 nw1310 nw1307 vdd vdd pch w=2u l=180n
M10880 nw1310 nw1306 vdd vdd pch w=2u l=180n
CT4131 t4131 0 0.1f
M10881 nw1310 nw1307 t4131 0 nch w=1u l=180n
M10882 t4131 nw1306 0 0 nch w=1u l=180n
Cnw1310 nw1310 0 2f
M10883 nw1311 nw1309 vdd vdd pch w=2u l=180n
M10884 nw1311 nw1310 vdd vdd pch w=2u l=180n
CT4132 t4132 0 0.1f
M10885 nw1311 nw1309 t4132 0 nch w=1u l=180n
M10886 t4132 nw1310 0 0 nch w=1u l=180n
Cnw1311 nw1311 0 2f
CT4133 t4133 0 0.1f
CT4134 t4134 0 0.1f
CT4135 t4135 0 0.1f
M10887 t4133 nw237 vdd vdd pch w=2u l=180n
M10888 t4133 nw1241 vdd vdd pch w=2u l=180n
CT4136 t4136 0 0.1f
M10889 t4133 nw237 t4136 0 nch w=1u l=180n
M10890 t4136 nw1241 0 0 nch w=1u l=180n
M10891 t4134 nw237 vdd vdd pch w=2u l=180n
M10892 t4134 t4133 vdd vdd pch w=2u l=180n
CT4137 t4137 0 0.1f
M10893 t4134 nw237 t4137 0 nch w=1u l=180n
M10894 t4137 t4133 0 0 nch w=1u l=180n
M10895 t4135 nw1241 vdd vdd pch w=2u l=180n
M10896 t4135 t4133 vdd vdd pch w=2u l=180n
CT4138 t4138 0 0.1f
M10897 t4135 nw1241 t4138 0 nch w=1u l=180n
M10898 t4138 t4133 0 0 nch w=1u l=180n
M10899 nw1312 t4134 vdd vdd pch w=2u l=180n
M10900 nw1312 t4135 vdd vdd pch w=2u l=180n
CT4139 t4139 0 0.1f
M10901 nw1312 t4134 t4139 0 nch w=1u l=180n
M10902 t4139 t4135 0 0 nch w=1u l=180n
Cnw1312 nw1312 0 2f
CT4140 t4140 0 0.1f
CT4141 t4141 0 0.1f
CT4142 t4142 0 0.1f
M10903 t4140 nw1312 vdd vdd pch w=2u l=180n
M10904 t4140 nw1311 vdd vdd pch w=2u l=180n
CT4143 t4143 0 0.1f
M10905 t4140 nw1312 t4143 0 nch w=1u l=180n
M10906 t4143 nw1311 0 0 nch w=1u l=180n
M10907 t4141 nw1312 vdd vdd pch w=2u l=180n
M10908 t4141 t4140 vdd vdd pch w=2u l=180n
CT4144 t4144 0 0.1f
M10909 t4141 nw1312 t4144 0 nch w=1u l=180n
M10910 t4144 t4140 0 0 nch w=1u l=180n
M10911 t4142 nw1311 vdd vdd pch w=2u l=180n
M10912 t4142 t4140 vdd vdd pch w=2u l=180n
CT4145 t4145 0 0.1f
M10913 t4142 nw1311 t4145 0 nch w=1u l=180n
M10914 t4145 t4140 0 0 nch w=1u l=180n
M10915 nw1313 t4141 vdd vdd pch w=2u l=180n
M10916 nw1313 t4142 vdd vdd pch w=2u l=180n
CT4146 t4146 0 0.1f
M10917 nw1313 t4141 t4146 0 nch w=1u l=180n
M10918 t4146 t4142 0 0 nch w=1u l=180n
Cnw1313 nw1313 0 2f
M10919 nw1314 nw237 vdd vdd pch w=2u l=180n
M10920 nw1314 nw1241 vdd vdd pch w=2u l=180n
CT4147 t4147 0 0.1f
M10921 nw1314 nw237 t4147 0 nch w=1u l=180n
M10922 t4147 nw1241 0 0 nch w=1u l=180n
Cnw1314 nw1314 0 2f
M10923 nw1315 nw1312 vdd vdd pch w=2u l=180n
M10924 nw1315 nw1311 vdd vdd pch w=2u l=180n
CT4148 t4148 0 0.1f
M10925 nw1315 nw1312 t4148 0 nch w=1u l=180n
M10926 t4148 nw1311 0 0 nch w=1u l=180n
Cnw1315 nw1315 0 2f
M10927 nw1316 nw1314 vdd vdd pch w=2u l=180n
M10928 nw1316 nw1315 vdd vdd pch w=2u l=180n
CT4149 t4149 0 0.1f
M10929 nw1316 nw1314 t4149 0 nch w=1u l=180n
M10930 t4149 nw1315 0 0 nch w=1u l=180n
Cnw1316 nw1316 0 2f
CT4150 t4150 0 0.1f
CT4151 t4151 0 0.1f
CT4152 t4152 0 0.1f
M10931 t4150 nw238 vdd vdd pch w=2u l=180n
M10932 t4150 nw1246 vdd vdd pch w=2u l=180n
CT4153 t4153 0 0.1f
M10933 t4150 nw238 t4153 0 nch w=1u l=180n
M10934 t4153 nw1246 0 0 nch w=1u l=180n
M10935 t4151 nw238 vdd vdd pch w=2u l=180n
M10936 t4151 t4150 vdd vdd pch w=2u l=180n
CT4154 t4154 0 0.1f
M10937 t4151 nw238 t4154 0 nch w=1u l=180n
M10938 t4154 t4150 0 0 nch w=1u l=180n
M10939 t4152 nw1246 vdd vdd pch w=2u l=180n
M10940 t4152 t4150 vdd vdd pch w=2u l=180n
CT4155 t4155 0 0.1f
M10941 t4152 nw1246 t4155 0 nch w=1u l=180n
M10942 t4155 t4150 0 0 nch w=1u l=180n
M10943 nw1317 t4151 vdd vdd pch w=2u l=180n
M10944 nw1317 t4152 vdd vdd pch w=2u l=180n
CT4156 t4156 0 0.1f
M10945 nw1317 t4151 t4156 0 nch w=1u l=180n
M10946 t4156 t4152 0 0 nch w=1u l=180n
Cnw1317 nw1317 0 2f
CT4157 t4157 0 0.1f
CT4158 t4158 0 0.1f
CT4159 t4159 0 0.1f
M10947 t4157 nw1317 vdd vdd pch w=2u l=180n
M10948 t4157 nw1316 vdd vdd pch w=2u l=180n
CT4160 t4160 0 0.1f
M10949 t4157 nw1317 t4160 0 nch w=1u l=180n
M10950 t4160 nw1316 0 0 nch w=1u l=180n
M10951 t4158 nw1317 vdd vdd pch w=2u l=180n
M10952 t4158 t4157 vdd vdd pch w=2u l=180n
CT4161 t4161 0 0.1f
M10953 t4158 nw1317 t4161 0 nch w=1u l=180n
M10954 t4161 t4157 0 0 nch w=1u l=180n
M10955 t4159 nw1316 vdd vdd pch w=2u l=180n
M10956 t4159 t4157 vdd vdd pch w=2u l=180n
CT4162 t4162 0 0.1f
M10957 t4159 nw1316 t4162 0 nch w=1u l=180n
M10958 t4162 t4157 0 0 nch w=1u l=180n
M10959 nw1318 t4158 vdd vdd pch w=2u l=180n
M10960 nw1318 t4159 vdd vdd pch w=2u l=180n
CT4163 t4163 0 0.1f
M10961 nw1318 t4158 t4163 0 nch w=1u l=180n
M10962 t4163 t4159 0 0 nch w=1u l=180n
Cnw1318 nw1318 0 2f
M10963 nw1319 nw238 vdd vdd pch w=2u l=180n
M10964 nw1319 nw1246 vdd vdd pch w=2u l=180n
CT4164 t4164 0 0.1f
M10965 nw1319 nw238 t4164 0 nch w=1u l=180n
M10966 t4164 nw1246 0 0 nch w=1u l=180n
Cnw1319 nw1319 0 2f
M10967 nw1320 nw1317 vdd vdd pch w=2u l=180n
M10968 nw1320 nw1316 vdd vdd pch w=2u l=180n
CT4165 t4165 0 0.1f
M10969 nw1320 nw1317 t4165 0 nch w=1u l=180n
M10970 t4165 nw1316 0 0 nch w=1u l=180n
Cnw1320 nw1320 0 2f
M10971 nw1321 nw1319 vdd vdd pch w=2u l=180n
M10972 nw1321 nw1320 vdd vdd pch w=2u l=180n
CT4166 t4166 0 0.1f
M10973 nw1321 nw1319 t4166 0 nch w=1u l=180n
M10974 t4166 nw1320 0 0 nch w=1u l=180n
Cnw1321 nw1321 0 2f
CT4167 t4167 0 0.1f
CT4168 t4168 0 0.1f
CT4169 t4169 0 0.1f
M10975 t4167 nw239 vdd vdd pch w=2u l=180n
M10976 t4167 nw1251 vdd vdd pch w=2u l=180n
CT4170 t4170 0 0.1f
M10977 t4167 nw239 t4170 0 nch w=1u l=180n
M10978 t4170 nw1251 0 0 nch w=1u l=180n
M10979 t4168 nw239 vdd vdd pch w=2u l=180n
M10980 t4168 t4167 vdd vdd pch w=2u l=180n
CT4171 t4171 0 0.1f
M10981 t4168 nw239 t4171 0 nch w=1u l=180n
M10982 t4171 t4167 0 0 nch w=1u l=180n
M10983 t4169 nw1251 vdd vdd pch w=2u l=180n
M10984 t4169 t4167 vdd vdd pch w=2u l=180n
CT4172 t4172 0 0.1f
M10985 t4169 nw1251 t4172 0 nch w=1u l=180n
M10986 t4172 t4167 0 0 nch w=1u l=180n
M10987 nw1322 t4168 vdd vdd pch w=2u l=180n
M10988 nw1322 t4169 vdd vdd pch w=2u l=180n
CT4173 t4173 0 0.1f
M10989 nw1322 t4168 t4173 0 nch w=1u l=180n
M10990 t4173 t4169 0 0 nch w=1u l=180n
Cnw1322 nw1322 0 2f
CT4174 t4174 0 0.1f
CT4175 t4175 0 0.1f
CT4176 t4176 0 0.1f
M10991 t4174 nw1322 vdd vdd pch w=2u l=180n
M10992 t4174 nw1321 vdd vdd pch w=2u l=180n
CT4177 t4177 0 0.1f
M10993 t4174 nw1322 t4177 0 nch w=1u l=180n
M10994 t4177 nw1321 0 0 nch w=1u l=180n
M10995 t4175 nw1322 vdd vdd pch w=2u l=180n
M10996 t4175 t4174 vdd vdd pch w=2u l=180n
CT4178 t4178 0 0.1f
M10997 t4175 nw1322 t4178 0 nch w=1u l=180n
M10998 t4178 t4174 0 0 nch w=1u l=180n
M10999 t4176 nw1321 vdd vdd pch w=2u l=180n
M11000 t4176 t4174 vdd vdd pch w=2u l=180n
CT4179 t4179 0 0.1f
M11001 t4176 nw1321 t4179 0 nch w=1u l=180n
M11002 t4179 t4174 0 0 nch w=1u l=180n
M11003 nw1323 t4175 vdd vdd pch w=2u l=180n
M11004 nw1323 t4176 vdd vdd pch w=2u l=180n
CT4180 t4180 0 0.1f
M11005 nw1323 t4175 t4180 0 nch w=1u l=180n
M11006 t4180 t4176 0 0 nch w=1u l=180n
Cnw1323 nw1323 0 2f
M11007 nw1324 nw239 vdd vdd pch w=2u l=180n
M11008 nw1324 nw1251 vdd vdd pch w=2u l=180n
CT4181 t4181 0 0.1f
M11009 nw1324 nw239 t4181 0 nch w=1u l=180n
M11010 t4181 nw1251 0 0 nch w=1u l=180n
Cnw1324 nw1324 0 2f
M11011 nw1325 nw1322 vdd vdd pch w=2u l=180n
M11012 nw1325 nw1321 vdd vdd pch w=2u l=180n
CT4182 t4182 0 0.1f
M11013 nw1325 nw1322 t4182 0 nch w=1u l=180n
M11014 t4182 nw1321 0 0 nch w=1u l=180n
Cnw1325 nw1325 0 2f
M11015 nw1326 nw1324 vdd vdd pch w=2u l=180n
M11016 nw1326 nw1325 vdd vdd pch w=2u l=180n
CT4183 t4183 0 0.1f
M11017 nw1326 nw1324 t4183 0 nch w=1u l=180n
M11018 t4183 nw1325 0 0 nch w=1u l=180n
Cnw1326 nw1326 0 2f
CT4184 t4184 0 0.1f
CT4185 t4185 0 0.1f
CT4186 t4186 0 0.1f
M11019 t4184 nw240 vdd vdd pch w=2u l=180n
M11020 t4184 nw1254 vdd vdd pch w=2u l=180n
CT4187 t4187 0 0.1f
M11021 t4184 nw240 t4187 0 nch w=1u l=180n
M11022 t4187 nw1254 0 0 nch w=1u l=180n
M11023 t4185 nw240 vdd vdd pch w=2u l=180n
M11024 t4185 t4184 vdd vdd pch w=2u l=180n
CT4188 t4188 0 0.1f
M11025 t4185 nw240 t4188 0 nch w=1u l=180n
M11026 t4188 t4184 0 0 nch w=1u l=180n
M11027 t4186 nw1254 vdd vdd pch w=2u l=180n
M11028 t4186 t4184 vdd vdd pch w=2u l=180n
CT4189 t4189 0 0.1f
M11029 t4186 nw1254 t4189 0 nch w=1u l=180n
M11030 t4189 t4184 0 0 nch w=1u l=180n
M11031 nw1327 t4185 vdd vdd pch w=2u l=180n
M11032 nw1327 t4186 vdd vdd pch w=2u l=180n
CT4190 t4190 0 0.1f
M11033 nw1327 t4185 t4190 0 nch w=1u l=180n
M11034 t4190 t4186 0 0 nch w=1u l=180n
Cnw1327 nw1327 0 2f
CT4191 t4191 0 0.1f
CT4192 t4192 0 0.1f
CT4193 t4193 0 0.1f
M11035 t4191 nw1327 vdd vdd pch w=2u l=180n
M11036 t4191 nw1326 vdd vdd pch w=2u l=180n
CT4194 t4194 0 0.1f
M11037 t4191 nw1327 t4194 0 nch w=1u l=180n
M11038 t4194 nw1326 0 0 nch w=1u l=180n
M11039 t4192 nw1327 vdd vdd pch w=2u l=180n
M11040 t4192 t4191 vdd vdd pch w=2u l=180n
CT4195 t4195 0 0.1f
M11041 t4192 nw1327 t4195 0 nch w=1u l=180n
M11042 t4195 t4191 0 0 nch w=1u l=180n
M11043 t4193 nw1326 vdd vdd pch w=2u l=180n
M11044 t4193 t4191 vdd vdd pch w=2u l=180n
CT4196 t4196 0 0.1f
M11045 t4193 nw1326 t4196 0 nch w=1u l=180n
M11046 t4196 t4191 0 0 nch w=1u l=180n
M11047 nw1328 t4192 vdd vdd pch w=2u l=180n
M11048 nw1328 t4193 vdd vdd pch w=2u l=180n
CT4197 t4197 0 0.1f
M11049 nw1328 t4192 t4197 0 nch w=1u l=180n
M11050 t4197 t4193 0 0 nch w=1u l=180n
Cnw1328 nw1328 0 2f
M11051 nw1329 nw240 vdd vdd pch w=2u l=180n
M11052 nw1329 nw1254 vdd vdd pch w=2u l=180n
CT4198 t4198 0 0.1f
M11053 nw1329 nw240 t4198 0 nch w=1u l=180n
M11054 t4198 nw1254 0 0 nch w=1u l=180n
Cnw1329 nw1329 0 2f
M11055 nw1330 nw1327 vdd vdd pch w=2u l=180n
M11056 nw1330 nw1326 vdd vdd pch w=2u l=180n
CT4199 t4199 0 0.1f
M11057 nw1330 nw1327 t4199 0 nch w=1u l=180n
M11058 t4199 nw1326 0 0 nch w=1u l=180n
Cnw1330 nw1330 0 2f
M11059 nw1331 nw1329 vdd vdd pch w=2u l=180n
M11060 nw1331 nw1330 vdd vdd pch w=2u l=180n
CT4200 t4200 0 0.1f
M11061 nw1331 nw1329 t4200 0 nch w=1u l=180n
M11062 t4200 nw1330 0 0 nch w=1u l=180n
Cnw1331 nw1331 0 2f
CT4201 t4201 0 0.1f
CT4202 t4202 0 0.1f
CT4203 t4203 0 0.1f
M11063 t4201 nw241 vdd vdd pch w=2u l=180n
M11064 t4201 nw1258 vdd vdd pch w=2u l=180n
CT4204 t4204 0 0.1f
M11065 t4201 nw241 t4204 0 nch w=1u l=180n
M11066 t4204 nw1258 0 0 nch w=1u l=180n
M11067 t4202 nw241 vdd vdd pch w=2u l=180n
M11068 t4202 t4201 vdd vdd pch w=2u l=180n
CT4205 t4205 0 0.1f
M11069 t4202 nw241 t4205 0 nch w=1u l=180n
M11070 t4205 t4201 0 0 nch w=1u l=180n
M11071 t4203 nw1258 vdd vdd pch w=2u l=180n
M11072 t4203 t4201 vdd vdd pch w=2u l=180n
CT4206 t4206 0 0.1f
M11073 t4203 nw1258 t4206 0 nch w=1u l=180n
M11074 t4206 t4201 0 0 nch w=1u l=180n
M11075 nw1332 t4202 vdd vdd pch w=2u l=180n
M11076 nw1332 t4203 vdd vdd pch w=2u l=180n
CT4207 t4207 0 0.1f
M11077 nw1332 t4202 t4207 0 nch w=1u l=180n
M11078 t4207 t4203 0 0 nch w=1u l=180n
Cnw1332 nw1332 0 2f
CT4208 t4208 0 0.1f
M11079 t4208 nw241 vdd vdd pch w=2u l=180n
M11080 t4208 nw1258 vdd vdd pch w=2u l=180n
CT4209 t4209 0 0.1f
M11081 t4208 nw241 t4209 0 nch w=1u l=180n
M11082 t4209 nw1258 0 0 nch w=1u l=180n
M11083 nw1333 t4208 vdd vdd pch w=2u l=180n
M11084 nw1333 t4208 0 0 nch w=1u l=180n
Cnw1333 nw1333 0 2f
CT4210 t4210 0 0.1f
CT4211 t4211 0 0.1f
CT4212 t4212 0 0.1f
M11085 t4210 nw242 vdd vdd pch w=2u l=180n
M11086 t4210 nw1263 vdd vdd pch w=2u l=180n
CT4213 t4213 0 0.1f
M11087 t4210 nw242 t4213 0 nch w=1u l=180n
M11088 t4213 nw1263 0 0 nch w=1u l=180n
M11089 t4211 nw242 vdd vdd pch w=2u l=180n
M11090 t4211 t4210 vdd vdd pch w=2u l=180n
CT4214 t4214 0 0.1f
M11091 t4211 nw242 t4214 0 nch w=1u l=180n
M11092 t4214 t4210 0 0 nch w=1u l=180n
M11093 t4212 nw1263 vdd vdd pch w=2u l=180n
M11094 t4212 t4210 vdd vdd pch w=2u l=180n
CT4215 t4215 0 0.1f
M11095 t4212 nw1263 t4215 0 nch w=1u l=180n
M11096 t4215 t4210 0 0 nch w=1u l=180n
M11097 nw1334 t4211 vdd vdd pch w=2u l=180n
M11098 nw1334 t4212 vdd vdd pch w=2u l=180n
CT4216 t4216 0 0.1f
M11099 nw1334 t4211 t4216 0 nch w=1u l=180n
M11100 t4216 t4212 0 0 nch w=1u l=180n
Cnw1334 nw1334 0 2f
CT4217 t4217 0 0.1f
CT4218 t4218 0 0.1f
CT4219 t4219 0 0.1f
M11101 t4217 nw1334 vdd vdd pch w=2u l=180n
M11102 t4217 nw1333 vdd vdd pch w=2u l=180n
CT4220 t4220 0 0.1f
M11103 t4217 nw1334 t4220 0 nch w=1u l=180n
M11104 t4220 nw1333 0 0 nch w=1u l=180n
M11105 t4218 nw1334 vdd vdd pch w=2u l=180n
M11106 t4218 t4217 vdd vdd pch w=2u l=180n
CT4221 t4221 0 0.1f
M11107 t4218 nw1334 t4221 0 nch w=1u l=180n
M11108 t4221 t4217 0 0 nch w=1u l=180n
M11109 t4219 nw1333 vdd vdd pch w=2u l=180n
M11110 t4219 t4217 vdd vdd pch w=2u l=180n
CT4222 t4222 0 0.1f
M11111 t4219 nw1333 t4222 0 nch w=1u l=180n
M11112 t4222 t4217 0 0 nch w=1u l=180n
M11113 nw1335 t4218 vdd vdd pch w=2u l=180n
M11114 nw1335 t4219 vdd vdd pch w=2u l=180n
CT4223 t4223 0 0.1f
M11115 nw1335 t4218 t4223 0 nch w=1u l=180n
M11116 t4223 t4219 0 0 nch w=1u l=180n
Cnw1335 nw1335 0 2f
M11117 nw1336 nw242 vdd vdd pch w=2u l=180n
M11118 nw1336 nw1263 vdd vdd pch w=2u l=180n
CT4224 t4224 0 0.1f
M11119 nw1336 nw242 t4224 0 nch w=1u l=180n
M11120 t4224 nw1263 0 0 nch w=1u l=180n
Cnw1336 nw1336 0 2f
M11121 nw1337 nw1334 vdd vdd pch w=2u l=180n
M11122 nw1337 nw1333 vdd vdd pch w=2u l=180n
CT4225 t4225 0 0.1f
M11123 nw1337 nw1334 t4225 0 nch w=1u l=180n
M11124 t4225 nw1333 0 0 nch w=1u l=180n
Cnw1337 nw1337 0 2f
M11125 nw1338 nw1336 vdd vdd pch w=2u l=180n
M11126 nw1338 nw1337 vdd vdd pch w=2u l=180n
CT4226 t4226 0 0.1f
M11127 nw1338 nw1336 t4226 0 nch w=1u l=180n
M11128 t4226 nw1337 0 0 nch w=1u l=180n
Cnw1338 nw1338 0 2f
CT4227 t4227 0 0.1f
CT4228 t4228 0 0.1f
CT4229 t4229 0 0.1f
M11129 t4227 nw243 vdd vdd pch w=2u l=180n
M11130 t4227 nw1268 vdd vdd pch w=2u l=180n
CT4230 t4230 0 0.1f
M11131 t4227 nw243 t4230 0 nch w=1u l=180n
M11132 t4230 nw1268 0 0 nch w=1u l=180n
M11133 t4228 nw243 vdd vdd pch w=2u l=180n
M11134 t4228 t4227 vdd vdd pch w=2u l=180n
CT4231 t4231 0 0.1f
M11135 t4228 nw243 t4231 0 nch w=1u l=180n
M11136 t4231 t4227 0 0 nch w=1u l=180n
M11137 t4229 nw1268 vdd vdd pch w=2u l=180n
M11138 t4229 t4227 vdd vdd pch w=2u l=180n
CT4232 t4232 0 0.1f
M11139 t4229 nw1268 t4232 0 nch w=1u l=180n
M11140 t4232 t4227 0 0 nch w=1u l=180n
M11141 nw1339 t4228 vdd vdd pch w=2u l=180n
M11142 nw1339 t4229 vdd vdd pch w=2u l=180n
CT4233 t4233 0 0.1f
M11143 nw1339 t4228 t4233 0 nch w=1u l=180n
M11144 t4233 t4229 0 0 nch w=1u l=180n
Cnw1339 nw1339 0 2f
CT4234 t4234 0 0.1f
CT4235 t4235 0 0.1f
CT4236 t4236 0 0.1f
M11145 t4234 nw1339 vdd vdd pch w=2u l=180n
M11146 t4234 nw1338 vdd vdd pch w=2u l=180n
CT4237 t4237 0 0.1f
M11147 t4234 nw1339 t4237 0 nch w=1u l=180n
M11148 t4237 nw1338 0 0 nch w=1u l=180n
M11149 t4235 nw1339 vdd vdd pch w=2u l=180n
M11150 t4235 t4234 vdd vdd pch w=2u l=180n
CT4238 t4238 0 0.1f
M11151 t4235 nw1339 t4238 0 nch w=1u l=180n
M11152 t4238 t4234 0 0 nch w=1u l=180n
M11153 t4236 nw1338 vdd vdd pch w=2u l=180n
M11154 t4236 t4234 vdd vdd pch w=2u l=180n
CT4239 t4239 0 0.1f
M11155 t4236 nw1338 t4239 0 nch w=1u l=180n
M11156 t4239 t4234 0 0 nch w=1u l=180n
M11157 nw1340 t4235 vdd vdd pch w=2u l=180n
M11158 nw1340 t4236 vdd vdd pch w=2u l=180n
CT4240 t4240 0 0.1f
M11159 nw1340 t4235 t4240 0 nch w=1u l=180n
M11160 t4240 t4236 0 0 nch w=1u l=180n
Cnw1340 nw1340 0 2f
M11161 nw1341 nw243 vdd vdd pch w=2u l=180n
M11162 nw1341 nw1268 vdd vdd pch w=2u l=180n
CT4241 t4241 0 0.1f
M11163 nw1341 nw243 t4241 0 nch w=1u l=180n
M11164 t4241 nw1268 0 0 nch w=1u l=180n
Cnw1341 nw1341 0 2f
M11165 nw1342 nw1339 vdd vdd pch w=2u l=180n
M11166 nw1342 nw1338 vdd vdd pch w=2u l=180n
CT4242 t4242 0 0.1f
M11167 nw1342 nw1339 t4242 0 nch w=1u l=180n
M11168 t4242 nw1338 0 0 nch w=1u l=180n
Cnw1342 nw1342 0 2f
M11169 nw1343 nw1341 vdd vdd pch w=2u l=180n
M11170 nw1343 nw1342 vdd vdd pch w=2u l=180n
CT4243 t4243 0 0.1f
M11171 nw1343 nw1341 t4243 0 nch w=1u l=180n
M11172 t4243 nw1342 0 0 nch w=1u l=180n
Cnw1343 nw1343 0 2f
CT4244 t4244 0 0.1f
CT4245 t4245 0 0.1f
CT4246 t4246 0 0.1f
M11173 t4244 nw244 vdd vdd pch w=2u l=180n
M11174 t4244 nw1273 vdd vdd pch w=2u l=180n
CT4247 t4247 0 0.1f
M11175 t4244 nw244 t4247 0 nch w=1u l=180n
M11176 t4247 nw1273 0 0 nch w=1u l=180n
M11177 t4245 nw244 vdd vdd pch w=2u l=180n
M11178 t4245 t4244 vdd vdd pch w=2u l=180n
CT4248 t4248 0 0.1f
M11179 t4245 nw244 t4248 0 nch w=1u l=180n
M11180 t4248 t4244 0 0 nch w=1u l=180n
M11181 t4246 nw1273 vdd vdd pch w=2u l=180n
M11182 t4246 t4244 vdd vdd pch w=2u l=180n
CT4249 t4249 0 0.1f
M11183 t4246 nw1273 t4249 0 nch w=1u l=180n
M11184 t4249 t4244 0 0 nch w=1u l=180n
M11185 nw1344 t4245 vdd vdd pch w=2u l=180n
M11186 nw1344 t4246 vdd vdd pch w=2u l=180n
CT4250 t4250 0 0.1f
M11187 nw1344 t4245 t4250 0 nch w=1u l=180n
M11188 t4250 t4246 0 0 nch w=1u l=180n
Cnw1344 nw1344 0 2f
CT4251 t4251 0 0.1f
CT4252 t4252 0 0.1f
CT4253 t4253 0 0.1f
M11189 t4251 nw1344 vdd vdd pch w=2u l=180n
M11190 t4251 nw1343 vdd vdd pch w=2u l=180n
CT4254 t4254 0 0.1f
M11191 t4251 nw1344 t4254 0 nch w=1u l=180n
M11192 t4254 nw1343 0 0 nch w=1u l=180n
M11193 t4252 nw1344 vdd vdd pch w=2u l=180n
M11194 t4252 t4251 vdd vdd pch w=2u l=180n
CT4255 t4255 0 0.1f
M11195 t4252 nw1344 t4255 0 nch w=1u l=180n
M11196 t4255 t4251 0 0 nch w=1u l=180n
M11197 t4253 nw1343 vdd vdd pch w=2u l=180n
M11198 t4253 t4251 vdd vdd pch w=2u l=180n
CT4256 t4256 0 0.1f
M11199 t4253 nw1343 t4256 0 nch w=1u l=180n
M11200 t4256 t4251 0 0 nch w=1u l=180n
M11201 nw1345 t4252 vdd vdd pch w=2u l=180n
M11202 nw1345 t4253 vdd vdd pch w=2u l=180n
CT4257 t4257 0 0.1f
M11203 nw1345 t4252 t4257 0 nch w=1u l=180n
M11204 t4257 t4253 0 0 nch w=1u l=180n
Cnw1345 nw1345 0 2f
M11205 nw1346 nw244 vdd vdd pch w=2u l=180n
M11206 nw1346 nw1273 vdd vdd pch w=2u l=180n
CT4258 t4258 0 0.1f
M11207 nw1346 nw244 t4258 0 nch w=1u l=180n
M11208 t4258 nw1273 0 0 nch w=1u l=180n
Cnw1346 nw1346 0 2f
M11209 nw1347 nw1344 vdd vdd pch w=2u l=180n
M11210 nw1347 nw1343 vdd vdd pch w=2u l=180n
CT4259 t4259 0 0.1f
M11211 nw1347 nw1344 t4259 0 nch w=1u l=180n
M11212 t4259 nw1343 0 0 nch w=1u l=180n
Cnw1347 nw1347 0 2f
M11213 nw1348 nw1346 vdd vdd pch w=2u l=180n
M11214 nw1348 nw1347 vdd vdd pch w=2u l=180n
CT4260 t4260 0 0.1f
M11215 nw1348 nw1346 t4260 0 nch w=1u l=180n
M11216 t4260 nw1347 0 0 nch w=1u l=180n
Cnw1348 nw1348 0 2f
CT4261 t4261 0 0.1f
CT4262 t4262 0 0.1f
CT4263 t4263 0 0.1f
M11217 t4261 nw245 vdd vdd pch w=2u l=180n
M11218 t4261 nw1278 vdd vdd pch w=2u l=180n
CT4264 t4264 0 0.1f
M11219 t4261 nw245 t4264 0 nch w=1u l=180n
M11220 t4264 nw1278 0 0 nch w=1u l=180n
M11221 t4262 nw245 vdd vdd pch w=2u l=180n
M11222 t4262 t4261 vdd vdd pch w=2u l=180n
CT4265 t4265 0 0.1f
M11223 t4262 nw245 t4265 0 nch w=1u l=180n
M11224 t4265 t4261 0 0 nch w=1u l=180n
M11225 t4263 nw1278 vdd vdd pch w=2u l=180n
M11226 t4263 t4261 vdd vdd pch w=2u l=180n
CT4266 t4266 0 0.1f
M11227 t4263 nw1278 t4266 0 nch w=1u l=180n
M11228 t4266 t4261 0 0 nch w=1u l=180n
M11229 nw1349 t4262 vdd vdd pch w=2u l=180n
M11230 nw1349 t4263 vdd vdd pch w=2u l=180n
CT4267 t4267 0 0.1f
M11231 nw1349 t4262 t4267 0 nch w=1u l=180n
M11232 t4267 t4263 0 0 nch w=1u l=180n
Cnw1349 nw1349 0 2f
CT4268 t4268 0 0.1f
CT4269 t4269 0 0.1f
CT4270 t4270 0 0.1f
M11233 t4268 nw1349 vdd vdd pch w=2u l=180n
M11234 t4268 nw1348 vdd vdd pch w=2u l=180n
CT4271 t4271 0 0.1f
M11235 t4268 nw1349 t4271 0 nch w=1u l=180n
M11236 t4271 nw1348 0 0 nch w=1u l=180n
M11237 t4269 nw1349 vdd vdd pch w=2u l=180n
M11238 t4269 t4268 vdd vdd pch w=2u l=180n
CT4272 t4272 0 0.1f
M11239 t4269 nw1349 t4272 0 nch w=1u l=180n
M11240 t4272 t4268 0 0 nch w=1u l=180n
M11241 t4270 nw1348 vdd vdd pch w=2u l=180n
M11242 t4270 t4268 vdd vdd pch w=2u l=180n
CT4273 t4273 0 0.1f
M11243 t4270 nw1348 t4273 0 nch w=1u l=180n
M11244 t4273 t4268 0 0 nch w=1u l=180n
M11245 nw1350 t4269 vdd vdd pch w=2u l=180n
M11246 nw1350 t4270 vdd vdd pch w=2u l=180n
CT4274 t4274 0 0.1f
M11247 nw1350 t4269 t4274 0 nch w=1u l=180n
M11248 t4274 t4270 0 0 nch w=1u l=180n
Cnw1350 nw1350 0 2f
M11249 nw1351 nw245 vdd vdd pch w=2u l=180n
M11250 nw1351 nw1278 vdd vdd pch w=2u l=180n
CT4275 t4275 0 0.1f
M11251 nw1351 nw245 t4275 0 nch w=1u l=180n
M11252 t4275 nw1278 0 0 nch w=1u l=180n
Cnw1351 nw1351 0 2f
M11253 nw1352 nw1349 vdd vdd pch w=2u l=180n
M11254 nw1352 nw1348 vdd vdd pch w=2u l=180n
CT4276 t4276 0 0.1f
M11255 nw1352 nw1349 t4276 0 nch w=1u l=180n
M11256 t4276 nw1348 0 0 nch w=1u l=180n
Cnw1352 nw1352 0 2f
M11257 nw1353 nw1351 vdd vdd pch w=2u l=180n
M11258 nw1353 nw1352 vdd vdd pch w=2u l=180n
CT4277 t4277 0 0.1f
M11259 nw1353 nw1351 t4277 0 nch w=1u l=180n
M11260 t4277 nw1352 0 0 nch w=1u l=180n
Cnw1353 nw1353 0 2f
CT4278 t4278 0 0.1f
CT4279 t4279 0 0.1f
CT4280 t4280 0 0.1f
M11261 t4278 nw246 vdd vdd pch w=2u l=180n
M11262 t4278 nw1283 vdd vdd pch w=2u l=180n
CT4281 t4281 0 0.1f
M11263 t4278 nw246 t4281 0 nch w=1u l=180n
M11264 t4281 nw1283 0 0 nch w=1u l=180n
M11265 t4279 nw246 vdd vdd pch w=2u l=180n
M11266 t4279 t4278 vdd vdd pch w=2u l=180n
CT4282 t4282 0 0.1f
M11267 t4279 nw246 t4282 0 nch w=1u l=180n
M11268 t4282 t4278 0 0 nch w=1u l=180n
M11269 t4280 nw1283 vdd vdd pch w=2u l=180n
M11270 t4280 t4278 vdd vdd pch w=2u l=180n
CT4283 t4283 0 0.1f
M11271 t4280 nw1283 t4283 0 nch w=1u l=180n
M11272 t4283 t4278 0 0 nch w=1u l=180n
M11273 nw1354 t4279 vdd vdd pch w=2u l=180n
M11274 nw1354 t4280 vdd vdd pch w=2u l=180n
CT4284 t4284 0 0.1f
M11275 nw1354 t4279 t4284 0 nch w=1u l=180n
M11276 t4284 t4280 0 0 nch w=1u l=180n
Cnw1354 nw1354 0 2f
CT4285 t4285 0 0.1f
CT4286 t4286 0 0.1f
CT4287 t4287 0 0.1f
M11277 t4285 nw1354 vdd vdd pch w=2u l=180n
M11278 t4285 nw1353 vdd vdd pch w=2u l=180n
CT4288 t4288 0 0.1f
M11279 t4285 nw1354 t4288 0 nch w=1u l=180n
M11280 t4288 nw1353 0 0 nch w=1u l=180n
M11281 t4286 nw1354 vdd vdd pch w=2u l=180n
M11282 t4286 t4285 vdd vdd pch w=2u l=180n
CT4289 t4289 0 0.1f
M11283 t4286 nw1354 t4289 0 nch w=1u l=180n
M11284 t4289 t4285 0 0 nch w=1u l=180n
M11285 t4287 nw1353 vdd vdd pch w=2u l=180n
M11286 t4287 t4285 vdd vdd pch w=2u l=180n
CT4290 t4290 0 0.1f
M11287 t4287 nw1353 t4290 0 nch w=1u l=180n
M11288 t4290 t4285 0 0 nch w=1u l=180n
M11289 nw1355 t4286 vdd vdd pch w=2u l=180n
M11290 nw1355 t4287 vdd vdd pch w=2u l=180n
CT4291 t4291 0 0.1f
M11291 nw1355 t4286 t4291 0 nch w=1u l=180n
M11292 t4291 t4287 0 0 nch w=1u l=180n
Cnw1355 nw1355 0 2f
M11293 nw1356 nw246 vdd vdd pch w=2u l=180n
M11294 nw1356 nw1283 vdd vdd pch w=2u l=180n
CT4292 t4292 0 0.1f
M11295 nw1356 nw246 t4292 0 nch w=1u l=180n
M11296 t4292 nw1283 0 0 nch w=1u l=180n
Cnw1356 nw1356 0 2f
M11297 nw1357 nw1354 vdd vdd pch w=2u l=180n
M11298 nw1357 nw1353 vdd vdd pch w=2u l=180n
CT4293 t4293 0 0.1f
M11299 nw1357 nw1354 t4293 0 nch w=1u l=180n
M11300 t4293 nw1353 0 0 nch w=1u l=180n
Cnw1357 nw1357 0 2f
M11301 nw1358 nw1356 vdd vdd pch w=2u l=180n
M11302 nw1358 nw1357 vdd vdd pch w=2u l=180n
CT4294 t4294 0 0.1f
M11303 nw1358 nw1356 t4294 0 nch w=1u l=180n
M11304 t4294 nw1357 0 0 nch w=1u l=180n
Cnw1358 nw1358 0 2f
CT4295 t4295 0 0.1f
CT4296 t4296 0 0.1f
CT4297 t4297 0 0.1f
M11305 t4295 nw247 vdd vdd pch w=2u l=180n
M11306 t4295 nw1288 vdd vdd pch w=2u l=180n
CT4298 t4298 0 0.1f
M11307 t4295 nw247 t4298 0 nch w=1u l=180n
M11308 t4298 nw1288 0 0 nch w=1u l=180n
M11309 t4296 nw247 vdd vdd pch w=2u l=180n
M11310 t4296 t4295 vdd vdd pch w=2u l=180n
CT4299 t4299 0 0.1f
M11311 t4296 nw247 t4299 0 nch w=1u l=180n
M11312 t4299 t4295 0 0 nch w=1u l=180n
M11313 t4297 nw1288 vdd vdd pch w=2u l=180n
M11314 t4297 t4295 vdd vdd pch w=2u l=180n
CT4300 t4300 0 0.1f
M11315 t4297 nw1288 t4300 0 nch w=1u l=180n
M11316 t4300 t4295 0 0 nch w=1u l=180n
M11317 nw1359 t4296 vdd vdd pch w=2u l=180n
M11318 nw1359 t4297 vdd vdd pch w=2u l=180n
CT4301 t4301 0 0.1f
M11319 nw1359 t4296 t4301 0 nch w=1u l=180n
M11320 t4301 t4297 0 0 nch w=1u l=180n
Cnw1359 nw1359 0 2f
CT4302 t4302 0 0.1f
CT4303 t4303 0 0.1f
CT4304 t4304 0 0.1f
M11321 t4302 nw1359 vdd vdd pch w=2u l=180n
M11322 t4302 nw1358 vdd vdd pch w=2u l=180n
CT4305 t4305 0 0.1f
M11323 t4302 nw1359 t4305 0 nch w=1u l=180n
M11324 t4305 nw1358 0 0 nch w=1u l=180n
M11325 t4303 nw1359 vdd vdd pch w=2u l=180n
M11326 t4303 t4302 vdd vdd pch w=2u l=180n
CT4306 t4306 0 0.1f
M11327 t4303 nw1359 t4306 0 nch w=1u l=180n
M11328 t4306 t4302 0 0 nch w=1u l=180n
M11329 t4304 nw1358 vdd vdd pch w=2u l=180n
M11330 t4304 t4302 vdd vdd pch w=2u l=180n
CT4307 t4307 0 0.1f
M11331 t4304 nw1358 t4307 0 nch w=1u l=180n
M11332 t4307 t4302 0 0 nch w=1u l=180n
M11333 nw1360 t4303 vdd vdd pch w=2u l=180n
M11334 nw1360 t4304 vdd vdd pch w=2u l=180n
CT4308 t4308 0 0.1f
M11335 nw1360 t4303 t4308 0 nch w=1u l=180n
M11336 t4308 t4304 0 0 nch w=1u l=180n
Cnw1360 nw1360 0 2f
M11337 nw1361 nw247 vdd vdd pch w=2u l=180n
M11338 nw1361 nw1288 vdd vdd pch w=2u l=180n
CT4309 t4309 0 0.1f
M11339 nw1361 nw247 t4309 0 nch w=1u l=180n
M11340 t4309 nw1288 0 0 nch w=1u l=180n
Cnw1361 nw1361 0 2f
M11341 nw1362 nw1359 vdd vdd pch w=2u l=180n
M11342 nw1362 nw1358 vdd vdd pch w=2u l=180n
CT4310 t4310 0 0.1f
M11343 nw1362 nw1359 t4310 0 nch w=1u l=180n
M11344 t4310 nw1358 0 0 nch w=1u l=180n
Cnw1362 nw1362 0 2f
M11345 nw1363 nw1361 vdd vdd pch w=2u l=180n
M11346 nw1363 nw1362 vdd vdd pch w=2u l=180n
CT4311 t4311 0 0.1f
M11347 nw1363 nw1361 t4311 0 nch w=1u l=180n
M11348 t4311 nw1362 0 0 nch w=1u l=180n
Cnw1363 nw1363 0 2f
CT4312 t4312 0 0.1f
CT4313 t4313 0 0.1f
CT4314 t4314 0 0.1f
M11349 t4312 nw248 vdd vdd pch w=2u l=180n
M11350 t4312 nw1293 vdd vdd pch w=2u l=180n
CT4315 t4315 0 0.1f
M11351 t4312 nw248 t4315 0 nch w=1u l=180n
M11352 t4315 nw1293 0 0 nch w=1u l=180n
M11353 t4313 nw248 vdd vdd pch w=2u l=180n
M11354 t4313 t4312 vdd vdd pch w=2u l=180n
CT4316 t4316 0 0.1f
M11355 t4313 nw248 t4316 0 nch w=1u l=180n
M11356 t4316 t4312 0 0 nch w=1u l=180n
M11357 t4314 nw1293 vdd vdd pch w=2u l=180n
M11358 t4314 t4312 vdd vdd pch w=2u l=180n
CT4317 t4317 0 0.1f
M11359 t4314 nw1293 t4317 0 nch w=1u l=180n
M11360 t4317 t4312 0 0 nch w=1u l=180n
M11361 nw1364 t4313 vdd vdd pch w=2u l=180n
M11362 nw1364 t4314 vdd vdd pch w=2u l=180n
CT4318 t4318 0 0.1f
M11363 nw1364 t4313 t4318 0 nch w=1u l=180n
M11364 t4318 t4314 0 0 nch w=1u l=180n
Cnw1364 nw1364 0 2f
CT4319 t4319 0 0.1f
CT4320 t4320 0 0.1f
CT4321 t4321 0 0.1f
M11365 t4319 nw1364 vdd vdd pch w=2u l=180n
M11366 t4319 nw1363 vdd vdd pch w=2u l=180n
CT4322 t4322 0 0.1f
M11367 t4319 nw1364 t4322 0 nch w=1u l=180n
M11368 t4322 nw1363 0 0 nch w=1u l=180n
M11369 t4320 nw1364 vdd vdd pch w=2u l=180n
M11370 t4320 t4319 vdd vdd pch w=2u l=180n
CT4323 t4323 0 0.1f
M11371 t4320 nw1364 t4323 0 nch w=1u l=180n
M11372 t4323 t4319 0 0 nch w=1u l=180n
M11373 t4321 nw1363 vdd vdd pch w=2u l=180n
M11374 t4321 t4319 vdd vdd pch w=2u l=180n
CT4324 t4324 0 0.1f
M11375 t4321 nw1363 t4324 0 nch w=1u l=180n
M11376 t4324 t4319 0 0 nch w=1u l=180n
M11377 nw1365 t4320 vdd vdd pch w=2u l=180n
M11378 nw1365 t4321 vdd vdd pch w=2u l=180n
CT4325 t4325 0 0.1f
M11379 nw1365 t4320 t4325 0 nch w=1u l=180n
M11380 t4325 t4321 0 0 nch w=1u l=180n
Cnw1365 nw1365 0 2f
M11381 nw1366 nw248 vdd vdd pch w=2u l=180n
M11382 nw1366 nw1293 vdd vdd pch w=2u l=180n
CT4326 t4326 0 0.1f
M11383 nw1366 nw248 t4326 0 nch w=1u l=180n
M11384 t4326 nw1293 0 0 nch w=1u l=180n
Cnw1366 nw1366 0 2f
M11385 nw1367 nw1364 vdd vdd pch w=2u l=180n
M11386 nw1367 nw1363 vdd vdd pch w=2u l=180n
CT4327 t4327 0 0.1f
M11387 nw1367 nw1364 t4327 0 nch w=1u l=180n
M11388 t4327 nw1363 0 0 nch w=1u l=180n
Cnw1367 nw1367 0 2f
M11389 nw1368 nw1366 vdd vdd pch w=2u l=180n
M11390 nw1368 nw1367 vdd vdd pch w=2u l=180n
CT4328 t4328 0 0.1f
M11391 nw1368 nw1366 t4328 0 nch w=1u l=180n
M11392 t4328 nw1367 0 0 nch w=1u l=180n
Cnw1368 nw1368 0 2f
CT4329 t4329 0 0.1f
CT4330 t4330 0 0.1f
CT4331 t4331 0 0.1f
M11393 t4329 nw249 vdd vdd pch w=2u l=180n
M11394 t4329 nw1298 vdd vdd pch w=2u l=180n
CT4332 t4332 0 0.1f
M11395 t4329 nw249 t4332 0 nch w=1u l=180n
M11396 t4332 nw1298 0 0 nch w=1u l=180n
M11397 t4330 nw249 vdd vdd pch w=2u l=180n
M11398 t4330 t4329 vdd vdd pch w=2u l=180n
CT4333 t4333 0 0.1f
M11399 t4330 nw249 t4333 0 nch w=1u l=180n
M11400 t4333 t4329 0 0 nch w=1u l=180n
M11401 t4331 nw1298 vdd vdd pch w=2u l=180n
M11402 t4331 t4329 vdd vdd pch w=2u l=180n
CT4334 t4334 0 0.1f
M11403 t4331 nw1298 t4334 0 nch w=1u l=180n
M11404 t4334 t4329 0 0 nch w=1u l=180n
M11405 nw1369 t4330 vdd vdd pch w=2u l=180n
M11406 nw1369 t4331 vdd vdd pch w=2u l=180n
CT4335 t4335 0 0.1f
M11407 nw1369 t4330 t4335 0 nch w=1u l=180n
M11408 t4335 t4331 0 0 nch w=1u l=180n
Cnw1369 nw1369 0 2f
CT4336 t4336 0 0.1f
CT4337 t4337 0 0.1f
CT4338 t4338 0 0.1f
M11409 t4336 nw1369 vdd vdd pch w=2u l=180n
M11410 t4336 nw1368 vdd vdd pch w=2u l=180n
CT4339 t4339 0 0.1f
M11411 t4336 nw1369 t4339 0 nch w=1u l=180n
M11412 t4339 nw1368 0 0 nch w=1u l=180n
M11413 t4337 nw1369 vdd vdd pch w=2u l=180n
M11414 t4337 t4336 vdd vdd pch w=2u l=180n
CT4340 t4340 0 0.1f
M11415 t4337 nw1369 t4340 0 nch w=1u l=180n
M11416 t4340 t4336 0 0 nch w=1u l=180n
M11417 t4338 nw1368 vdd vdd pch w=2u l=180n
M11418 t4338 t4336 vdd vdd pch w=2u l=180n
CT4341 t4341 0 0.1f
M11419 t4338 nw1368 t4341 0 nch w=1u l=180n
M11420 t4341 t4336 0 0 nch w=1u l=180n
M11421 nw1370 t4337 vdd vdd pch w=2u l=180n
M11422 nw1370 t4338 vdd vdd pch w=2u l=180n
CT4342 t4342 0 0.1f
M11423 nw1370 t4337 t4342 0 nch w=1u l=180n
M11424 t4342 t4338 0 0 nch w=1u l=180n
Cnw1370 nw1370 0 2f
M11425 nw1371 nw249 vdd vdd pch w=2u l=180n
M11426 nw1371 nw1298 vdd vdd pch w=2u l=180n
CT4343 t4343 0 0.1f
M11427 nw1371 nw249 t4343 0 nch w=1u l=180n
M11428 t4343 nw1298 0 0 nch w=1u l=180n
Cnw1371 nw1371 0 2f
M11429 nw1372 nw1369 vdd vdd pch w=2u l=180n
M11430 nw1372 nw1368 vdd vdd pch w=2u l=180n
CT4344 t4344 0 0.1f
M11431 nw1372 nw1369 t4344 0 nch w=1u l=180n
M11432 t4344 nw1368 0 0 nch w=1u l=180n
Cnw1372 nw1372 0 2f
M11433 nw1373 nw1371 vdd vdd pch w=2u l=180n
M11434 nw1373 nw1372 vdd vdd pch w=2u l=180n
CT4345 t4345 0 0.1f
M11435 nw1373 nw1371 t4345 0 nch w=1u l=180n
M11436 t4345 nw1372 0 0 nch w=1u l=180n
Cnw1373 nw1373 0 2f
CT4346 t4346 0 0.1f
CT4347 t4347 0 0.1f
CT4348 t4348 0 0.1f
M11437 t4346 nw250 vdd vdd pch w=2u l=180n
M11438 t4346 nw1303 vdd vdd pch w=2u l=180n
CT4349 t4349 0 0.1f
M11439 t4346 nw250 t4349 0 nch w=1u l=180n
M11440 t4349 nw1303 0 0 nch w=1u l=180n
M11441 t4347 nw250 vdd vdd pch w=2u l=180n
M11442 t4347 t4346 vdd vdd pch w=2u l=180n
CT4350 t4350 0 0.1f
M11443 t4347 nw250 t4350 0 nch w=1u l=180n
M11444 t4350 t4346 0 0 nch w=1u l=180n
M11445 t4348 nw1303 vdd vdd pch w=2u l=180n
M11446 t4348 t4346 vdd vdd pch w=2u l=180n
CT4351 t4351 0 0.1f
M11447 t4348 nw1303 t4351 0 nch w=1u l=180n
M11448 t4351 t4346 0 0 nch w=1u l=180n
M11449 nw1374 t4347 vdd vdd pch w=2u l=180n
M11450 nw1374 t4348 vdd vdd pch w=2u l=180n
CT4352 t4352 0 0.1f
M11451 nw1374 t4347 t4352 0 nch w=1u l=180n
M11452 t4352 t4348 0 0 nch w=1u l=180n
Cnw1374 nw1374 0 2f
CT4353 t4353 0 0.1f
CT4354 t4354 0 0.1f
CT4355 t4355 0 0.1f
M11453 t4353 nw1374 vdd vdd pch w=2u l=180n
M11454 t4353 nw1373 vdd vdd pch w=2u l=180n
CT4356 t4356 0 0.1f
M11455 t4353 nw1374 t4356 0 nch w=1u l=180n
M11456 t4356 nw1373 0 0 nch w=1u l=180n
M11457 t4354 nw1374 vdd vdd pch w=2u l=180n
M11458 t4354 t4353 vdd vdd pch w=2u l=180n
CT4357 t4357 0 0.1f
M11459 t4354 nw1374 t4357 0 nch w=1u l=180n
M11460 t4357 t4353 0 0 nch w=1u l=180n
M11461 t4355 nw1373 vdd vdd pch w=2u l=180n
M11462 t4355 t4353 vdd vdd pch w=2u l=180n
CT4358 t4358 0 0.1f
M11463 t4355 nw1373 t4358 0 nch w=1u l=180n
M11464 t4358 t4353 0 0 nch w=1u l=180n
M11465 nw1375 t4354 vdd vdd pch w=2u l=180n
M11466 nw1375 t4355 vdd vdd pch w=2u l=180n
CT4359 t4359 0 0.1f
M11467 nw1375 t4354 t4359 0 nch w=1u l=180n
M11468 t4359 t4355 0 0 nch w=1u l=180n
Cnw1375 nw1375 0 2f
M11469 nw1376 nw250 vdd vdd pch w=2u l=180n
M11470 nw1376 nw1303 vdd vdd pch w=2u l=180n
CT4360 t4360 0 0.1f
M11471 nw1376 nw250 t4360 0 nch w=1u l=180n
M11472 t4360 nw1303 0 0 nch w=1u l=180n
Cnw1376 nw1376 0 2f
M11473 nw1377 nw1374 vdd vdd pch w=2u l=180n
M11474 nw1377 nw1373 vdd vdd pch w=2u l=180n
CT4361 t4361 0 0.1f
M11475 nw1377 nw1374 t4361 0 nch w=1u l=180n
M11476 t4361 nw1373 0 0 nch w=1u l=180n
Cnw1377 nw1377 0 2f
M11477 nw1378 nw1376 vdd vdd pch w=2u l=180n
M11478 nw1378 nw1377 vdd vdd pch w=2u l=180n
CT4362 t4362 0 0.1f
M11479 nw1378 nw1376 t4362 0 nch w=1u l=180n
M11480 t4362 nw1377 0 0 nch w=1u l=180n
Cnw1378 nw1378 0 2f
CT4363 t4363 0 0.1f
CT4364 t4364 0 0.1f
CT4365 t4365 0 0.1f
M11481 t4363 nw251 vdd vdd pch w=2u l=180n
M11482 t4363 nw1308 vdd vdd pch w=2u l=180n
CT4366 t4366 0 0.1f
M11483 t4363 nw251 t4366 0 nch w=1u l=180n
M11484 t4366 nw1308 0 0 nch w=1u l=180n
M11485 t4364 nw251 vdd vdd pch w=2u l=180n
M11486 t4364 t4363 vdd vdd pch w=2u l=180n
CT4367 t4367 0 0.1f
M11487 t4364 nw251 t4367 0 nch w=1u l=180n
M11488 t4367 t4363 0 0 nch w=1u l=180n
M11489 t4365 nw1308 vdd vdd pch w=2u l=180n
M11490 t4365 t4363 vdd vdd pch w=2u l=180n
CT4368 t4368 0 0.1f
M11491 t4365 nw1308 t4368 0 nch w=1u l=180n
M11492 t4368 t4363 0 0 nch w=1u l=180n
M11493 nw1379 t4364 vdd vdd pch w=2u l=180n
M11494 nw1379 t4365 vdd vdd pch w=2u l=180n
CT4369 t4369 0 0.1f
M11495 nw1379 t4364 t4369 0 nch w=1u l=180n
M11496 t4369 t4365 0 0 nch w=1u l=180n
Cnw1379 nw1379 0 2f
CT4370 t4370 0 0.1f
CT4371 t4371 0 0.1f
CT4372 t4372 0 0.1f
M11497 t4370 nw1379 vdd vdd pch w=2u l=180n
M11498 t4370 nw1378 vdd vdd pch w=2u l=180n
CT4373 t4373 0 0.1f
M11499 t4370 nw1379 t4373 0 nch w=1u l=180n
M11500 t4373 nw1378 0 0 nch w=1u l=180n
M11501 t4371 nw1379 vdd vdd pch w=2u l=180n
M11502 t4371 t4370 vdd vdd pch w=2u l=180n
CT4374 t4374 0 0.1f
M11503 t4371 nw1379 t4374 0 nch w=1u l=180n
M11504 t4374 t4370 0 0 nch w=1u l=180n
M11505 t4372 nw1378 vdd vdd pch w=2u l=180n
M11506 t4372 t4370 vdd vdd pch w=2u l=180n
CT4375 t4375 0 0.1f
M11507 t4372 nw1378 t4375 0 nch w=1u l=180n
M11508 t4375 t4370 0 0 nch w=1u l=180n
M11509 nw1380 t4371 vdd vdd pch w=2u l=180n
M11510 nw1380 t4372 vdd vdd pch w=2u l=180n
CT4376 t4376 0 0.1f
M11511 nw1380 t4371 t4376 0 nch w=1u l=180n
M11512 t4376 t4372 0 0 nch w=1u l=180n
Cnw1380 nw1380 0 2f
M11513 nw1381 nw251 vdd vdd pch w=2u l=180n
M11514 nw1381 nw1308 vdd vdd pch w=2u l=180n
CT4377 t4377 0 0.1f
M11515 nw1381 nw251 t4377 0 nch w=1u l=180n
M11516 t4377 nw1308 0 0 nch w=1u l=180n
Cnw1381 nw1381 0 2f
M11517 nw1382 nw1379 vdd vdd pch w=2u l=180n
M11518 nw1382 nw1378 vdd vdd pch w=2u l=180n
CT4378 t4378 0 0.1f
M11519 nw1382 nw1379 t4378 0 nch w=1u l=180n
M11520 t4378 nw1378 0 0 nch w=1u l=180n
Cnw1382 nw1382 0 2f
M11521 nw1383 nw1381 vdd vdd pch w=2u l=180n
M11522 nw1383 nw1382 vdd vdd pch w=2u l=180n
CT4379 t4379 0 0.1f
M11523 nw1383 nw1381 t4379 0 nch w=1u l=180n
M11524 t4379 nw1382 0 0 nch w=1u l=180n
Cnw1383 nw1383 0 2f
CT4380 t4380 0 0.1f
CT4381 t4381 0 0.1f
CT4382 t4382 0 0.1f
M11525 t4380 nw252 vdd vdd pch w=2u l=180n
M11526 t4380 nw1313 vdd vdd pch w=2u l=180n
CT4383 t4383 0 0.1f
M11527 t4380 nw252 t4383 0 nch w=1u l=180n
M11528 t4383 nw1313 0 0 nch w=1u l=180n
M11529 t4381 nw252 vdd vdd pch w=2u l=180n
M11530 t4381 t4380 vdd vdd pch w=2u l=180n
CT4384 t4384 0 0.1f
M11531 t4381 nw252 t4384 0 nch w=1u l=180n
M11532 t4384 t4380 0 0 nch w=1u l=180n
M11533 t4382 nw1313 vdd vdd pch w=2u l=180n
M11534 t4382 t4380 vdd vdd pch w=2u l=180n
CT4385 t4385 0 0.1f
M11535 t4382 nw1313 t4385 0 nch w=1u l=180n
M11536 t4385 t4380 0 0 nch w=1u l=180n
M11537 nw1384 t4381 vdd vdd pch w=2u l=180n
M11538 nw1384 t4382 vdd vdd pch w=2u l=180n
CT4386 t4386 0 0.1f
M11539 nw1384 t4381 t4386 0 nch w=1u l=180n
M11540 t4386 t4382 0 0 nch w=1u l=180n
Cnw1384 nw1384 0 2f
CT4387 t4387 0 0.1f
CT4388 t4388 0 0.1f
CT4389 t4389 0 0.1f
M11541 t4387 nw1384 vdd vdd pch w=2u l=180n
M11542 t4387 nw1383 vdd vdd pch w=2u l=180n
CT4390 t4390 0 0.1f
M11543 t4387 nw1384 t4390 0 nch w=1u l=180n
M11544 t4390 nw1383 0 0 nch w=1u l=180n
M11545 t4388 nw1384 vdd vdd pch w=2u l=180n
M11546 t4388 t4387 vdd vdd pch w=2u l=180n
CT4391 t4391 0 0.1f
M11547 t4388 nw1384 t4391 0 nch w=1u l=180n
M11548 t4391 t4387 0 0 nch w=1u l=180n
M11549 t4389 nw1383 vdd vdd pch w=2u l=180n
M11550 t4389 t4387 vdd vdd pch w=2u l=180n
CT4392 t4392 0 0.1f
M11551 t4389 nw1383 t4392 0 nch w=1u l=180n
M11552 t4392 t4387 0 0 nch w=1u l=180n
M11553 nw1385 t4388 vdd vdd pch w=2u l=180n
M11554 nw1385 t4389 vdd vdd pch w=2u l=180n
CT4393 t4393 0 0.1f
M11555 nw1385 t4388 t4393 0 nch w=1u l=180n
M11556 t4393 t4389 0 0 nch w=1u l=180n
Cnw1385 nw1385 0 2f
M11557 nw1386 nw252 vdd vdd pch w=2u l=180n
M11558 nw1386 nw1313 vdd vdd pch w=2u l=180n
CT4394 t4394 0 0.1f
M11559 nw1386 nw252 t4394 0 nch w=1u l=180n
M11560 t4394 nw1313 0 0 nch w=1u l=180n
Cnw1386 nw1386 0 2f
M11561 nw1387 nw1384 vdd vdd pch w=2u l=180n
M11562 nw1387 nw1383 vdd vdd pch w=2u l=180n
CT4395 t4395 0 0.1f
M11563 nw1387 nw1384 t4395 0 nch w=1u l=180n
M11564 t4395 nw1383 0 0 nch w=1u l=180n
Cnw1387 nw1387 0 2f
M11565 nw1388 nw1386 vdd vdd pch w=2u l=180n
M11566 nw1388 nw1387 vdd vdd pch w=2u l=180n
CT4396 t4396 0 0.1f
M11567 nw1388 nw1386 t4396 0 nch w=1u l=180n
M11568 t4396 nw1387 0 0 nch w=1u l=180n
Cnw1388 nw1388 0 2f
CT4397 t4397 0 0.1f
CT4398 t4398 0 0.1f
CT4399 t4399 0 0.1f
M11569 t4397 nw253 vdd vdd pch w=2u l=180n
M11570 t4397 nw1318 vdd vdd pch w=2u l=180n
CT4400 t4400 0 0.1f
M11571 t4397 nw253 t4400 0 nch w=1u l=180n
M11572 t4400 nw1318 0 0 nch w=1u l=180n
M11573 t4398 nw253 vdd vdd pch w=2u l=180n
M11574 t4398 t4397 vdd vdd pch w=2u l=180n
CT4401 t4401 0 0.1f
M11575 t4398 nw253 t4401 0 nch w=1u l=180n
M11576 t4401 t4397 0 0 nch w=1u l=180n
M11577 t4399 nw1318 vdd vdd pch w=2u l=180n
M11578 t4399 t4397 vdd vdd pch w=2u l=180n
CT4402 t4402 0 0.1f
M11579 t4399 nw1318 t4402 0 nch w=1u l=180n
M11580 t4402 t4397 0 0 nch w=1u l=180n
M11581 nw1389 t4398 vdd vdd pch w=2u l=180n
M11582 nw1389 t4399 vdd vdd pch w=2u l=180n
CT4403 t4403 0 0.1f
M11583 nw1389 t4398 t4403 0 nch w=1u l=180n
M11584 t4403 t4399 0 0 nch w=1u l=180n
Cnw1389 nw1389 0 2f
CT4404 t4404 0 0.1f
CT4405 t4405 0 0.1f
CT4406 t4406 0 0.1f
M11585 t4404 nw1389 vdd vdd pch w=2u l=180n
M11586 t4404 nw1388 vdd vdd pch w=2u l=180n
CT4407 t4407 0 0.1f
M11587 t4404 nw1389 t4407 0 nch w=1u l=180n
M11588 t4407 nw1388 0 0 nch w=1u l=180n
M11589 t4405 nw1389 vdd vdd pch w=2u l=180n
M11590 t4405 t4404 vdd vdd pch w=2u l=180n
CT4408 t4408 0 0.1f
M11591 t4405 nw1389 t4408 0 nch w=1u l=180n
M11592 t4408 t4404 0 0 nch w=1u l=180n
M11593 t4406 nw1388 vdd vdd pch w=2u l=180n
M11594 t4406 t4404 vdd vdd pch w=2u l=180n
CT4409 t4409 0 0.1f
M11595 t4406 nw1388 t4409 0 nch w=1u l=180n
M11596 t4409 t4404 0 0 nch w=1u l=180n
M11597 nw1390 t4405 vdd vdd pch w=2u l=180n
M11598 nw1390 t4406 vdd vdd pch w=2u l=180n
CT4410 t4410 0 0.1f
M11599 nw1390 t4405 t4410 0 nch w=1u l=180n
M11600 t4410 t4406 0 0 nch w=1u l=180n
Cnw1390 nw1390 0 2f
M11601 nw1391 nw253 vdd vdd pch w=2u l=180n
M11602 nw1391 nw1318 vdd vdd pch w=2u l=180n
CT4411 t4411 0 0.1f
M11603 nw1391 nw253 t4411 0 nch w=1u l=180n
M11604 t4411 nw1318 0 0 nch w=1u l=180n
Cnw1391 nw1391 0 2f
M11605 nw1392 nw1389 vdd vdd pch w=2u l=180n
M11606 nw1392 nw1388 vdd vdd pch w=2u l=180n
CT4412 t4412 0 0.1f
M11607 nw1392 nw1389 t4412 0 nch w=1u l=180n
M11608 t4412 nw1388 0 0 nch w=1u l=180n
Cnw1392 nw1392 0 2f
M11609 nw1393 nw1391 vdd vdd pch w=2u l=180n
M11610 nw1393 nw1392 vdd vdd pch w=2u l=180n
CT4413 t4413 0 0.1f
M11611 nw1393 nw1391 t4413 0 nch w=1u l=180n
M11612 t4413 nw1392 0 0 nch w=1u l=180n
Cnw1393 nw1393 0 2f
CT4414 t4414 0 0.1f
CT4415 t4415 0 0.1f
CT4416 t4416 0 0.1f
M11613 t4414 nw254 vdd vdd pch w=2u l=180n
M11614 t4414 nw1323 vdd vdd pch w=2u l=180n
CT4417 t4417 0 0.1f
M11615 t4414 nw254 t4417 0 nch w=1u l=180n
M11616 t4417 nw1323 0 0 nch w=1u l=180n
M11617 t4415 nw254 vdd vdd pch w=2u l=180n
M11618 t4415 t4414 vdd vdd pch w=2u l=180n
CT4418 t4418 0 0.1f
M11619 t4415 nw254 t4418 0 nch w=1u l=180n
M11620 t4418 t4414 0 0 nch w=1u l=180n
M11621 t4416 nw1323 vdd vdd pch w=2u l=180n
M11622 t4416 t4414 vdd vdd pch w=2u l=180n
CT4419 t4419 0 0.1f
M11623 t4416 nw1323 t4419 0 nch w=1u l=180n
M11624 t4419 t4414 0 0 nch w=1u l=180n
M11625 nw1394 t4415 vdd vdd pch w=2u l=180n
M11626 nw1394 t4416 vdd vdd pch w=2u l=180n
CT4420 t4420 0 0.1f
M11627 nw1394 t4415 t4420 0 nch w=1u l=180n
M11628 t4420 t4416 0 0 nch w=1u l=180n
Cnw1394 nw1394 0 2f
CT4421 t4421 0 0.1f
CT4422 t4422 0 0.1f
CT4423 t4423 0 0.1f
M11629 t4421 nw1394 vdd vdd pch w=2u l=180n
M11630 t4421 nw1393 vdd vdd pch w=2u l=180n
CT4424 t4424 0 0.1f
M11631 t4421 nw1394 t4424 0 nch w=1u l=180n
M11632 t4424 nw1393 0 0 nch w=1u l=180n
M11633 t4422 nw1394 vdd vdd pch w=2u l=180n
M11634 t4422 t4421 vdd vdd pch w=2u l=180n
CT4425 t4425 0 0.1f
M11635 t4422 nw1394 t4425 0 nch w=1u l=180n
M11636 t4425 t4421 0 0 nch w=1u l=180n
M11637 t4423 nw1393 vdd vdd pch w=2u l=180n
M11638 t4423 t4421 vdd vdd pch w=2u l=180n
CT4426 t4426 0 0.1f
M11639 t4423 nw1393 t4426 0 nch w=1u l=180n
M11640 t4426 t4421 0 0 nch w=1u l=180n
M11641 nw1395 t4422 vdd vdd pch w=2u l=180n
M11642 nw1395 t4423 vdd vdd pch w=2u l=180n
CT4427 t4427 0 0.1f
M11643 nw1395 t4422 t4427 0 nch w=1u l=180n
M11644 t4427 t4423 0 0 nch w=1u l=180n
Cnw1395 nw1395 0 2f
M11645 nw1396 nw254 vdd vdd pch w=2u l=180n
M11646 nw1396 nw1323 vdd vdd pch w=2u l=180n
CT4428 t4428 0 0.1f
M11647 nw1396 nw254 t4428 0 nch w=1u l=180n
M11648 t4428 nw1323 0 0 nch w=1u l=180n
Cnw1396 nw1396 0 2f
M11649 nw1397 nw1394 vdd vdd pch w=2u l=180n
M11650 nw1397 nw1393 vdd vdd pch w=2u l=180n
CT4429 t4429 0 0.1f
M11651 nw1397 nw1394 t4429 0 nch w=1u l=180n
M11652 t4429 nw1393 0 0 nch w=1u l=180n
Cnw1397 nw1397 0 2f
M11653 nw1398 nw1396 vdd vdd pch w=2u l=180n
M11654 nw1398 nw1397 vdd vdd pch w=2u l=180n
CT4430 t4430 0 0.1f
M11655 nw1398 nw1396 t4430 0 nch w=1u l=180n
M11656 t4430 nw1397 0 0 nch w=1u l=180n
Cnw1398 nw1398 0 2f
CT4431 t4431 0 0.1f
CT4432 t4432 0 0.1f
CT4433 t4433 0 0.1f
M11657 t4431 nw255 vdd vdd pch w=2u l=180n
M11658 t4431 nw1328 vdd vdd pch w=2u l=180n
CT4434 t4434 0 0.1f
M11659 t4431 nw255 t4434 0 nch w=1u l=180n
M11660 t4434 nw1328 0 0 nch w=1u l=180n
M11661 t4432 nw255 vdd vdd pch w=2u l=180n
M11662 t4432 t4431 vdd vdd pch w=2u l=180n
CT4435 t4435 0 0.1f
M11663 t4432 nw255 t4435 0 nch w=1u l=180n
M11664 t4435 t4431 0 0 nch w=1u l=180n
M11665 t4433 nw1328 vdd vdd pch w=2u l=180n
M11666 t4433 t4431 vdd vdd pch w=2u l=180n
CT4436 t4436 0 0.1f
M11667 t4433 nw1328 t4436 0 nch w=1u l=180n
M11668 t4436 t4431 0 0 nch w=1u l=180n
M11669 nw1399 t4432 vdd vdd pch w=2u l=180n
M11670 nw1399 t4433 vdd vdd pch w=2u l=180n
CT4437 t4437 0 0.1f
M11671 nw1399 t4432 t4437 0 nch w=1u l=180n
M11672 t4437 t4433 0 0 nch w=1u l=180n
Cnw1399 nw1399 0 2f
CT4438 t4438 0 0.1f
CT4439 t4439 0 0.1f
CT4440 t4440 0 0.1f
M11673 t4438 nw1399 vdd vdd pch w=2u l=180n
M11674 t4438 nw1398 vdd vdd pch w=2u l=180n
CT4441 t4441 0 0.1f
M11675 t4438 nw1399 t4441 0 nch w=1u l=180n
M11676 t4441 nw1398 0 0 nch w=1u l=180n
M11677 t4439 nw1399 vdd vdd pch w=2u l=180n
M11678 t4439 t4438 vdd vdd pch w=2u l=180n
CT4442 t4442 0 0.1f
M11679 t4439 nw1399 t4442 0 nch w=1u l=180n
M11680 t4442 t4438 0 0 nch w=1u l=180n
M11681 t4440 nw1398 vdd vdd pch w=2u l=180n
M11682 t4440 t4438 vdd vdd pch w=2u l=180n
CT4443 t4443 0 0.1f
M11683 t4440 nw1398 t4443 0 nch w=1u l=180n
M11684 t4443 t4438 0 0 nch w=1u l=180n
M11685 nw1400 t4439 vdd vdd pch w=2u l=180n
M11686 nw1400 t4440 vdd vdd pch w=2u l=180n
CT4444 t4444 0 0.1f
M11687 nw1400 t4439 t4444 0 nch w=1u l=180n
M11688 t4444 t4440 0 0 nch w=1u l=180n
Cnw1400 nw1400 0 2f
M11689 nw1401 nw255 vdd vdd pch w=2u l=180n
M11690 nw1401 nw1328 vdd vdd pch w=2u l=180n
CT4445 t4445 0 0.1f
M11691 nw1401 nw255 t4445 0 nch w=1u l=180n
M11692 t4445 nw1328 0 0 nch w=1u l=180n
Cnw1401 nw1401 0 2f
M11693 nw1402 nw1399 vdd vdd pch w=2u l=180n
M11694 nw1402 nw1398 vdd vdd pch w=2u l=180n
CT4446 t4446 0 0.1f
M11695 nw1402 nw1399 t4446 0 nch w=1u l=180n
M11696 t4446 nw1398 0 0 nch w=1u l=180n
Cnw1402 nw1402 0 2f
M11697 nw1403 nw1401 vdd vdd pch w=2u l=180n
M11698 nw1403 nw1402 vdd vdd pch w=2u l=180n
CT4447 t4447 0 0.1f
M11699 nw1403 nw1401 t4447 0 nch w=1u l=180n
M11700 t4447 nw1402 0 0 nch w=1u l=180n
Cnw1403 nw1403 0 2f
CT4448 t4448 0 0.1f
CT4449 t4449 0 0.1f
CT4450 t4450 0 0.1f
M11701 t4448 nw256 vdd vdd pch w=2u l=180n
M11702 t4448 nw1331 vdd vdd pch w=2u l=180n
CT4451 t4451 0 0.1f
M11703 t4448 nw256 t4451 0 nch w=1u l=180n
M11704 t4451 nw1331 0 0 nch w=1u l=180n
M11705 t4449 nw256 vdd vdd pch w=2u l=180n
M11706 t4449 t4448 vdd vdd pch w=2u l=180n
CT4452 t4452 0 0.1f
M11707 t4449 nw256 t4452 0 nch w=1u l=180n
M11708 t4452 t4448 0 0 nch w=1u l=180n
M11709 t4450 nw1331 vdd vdd pch w=2u l=180n
M11710 t4450 t4448 vdd vdd pch w=2u l=180n
CT4453 t4453 0 0.1f
M11711 t4450 nw1331 t4453 0 nch w=1u l=180n
M11712 t4453 t4448 0 0 nch w=1u l=180n
M11713 nw1404 t4449 vdd vdd pch w=2u l=180n
M11714 nw1404 t4450 vdd vdd pch w=2u l=180n
CT4454 t4454 0 0.1f
M11715 nw1404 t4449 t4454 0 nch w=1u l=180n
M11716 t4454 t4450 0 0 nch w=1u l=180n
Cnw1404 nw1404 0 2f
CT4455 t4455 0 0.1f
CT4456 t4456 0 0.1f
CT4457 t4457 0 0.1f
M11717 t4455 nw1404 vdd vdd pch w=2u l=180n
M11718 t4455 nw1403 vdd vdd pch w=2u l=180n
CT4458 t4458 0 0.1f
M11719 t4455 nw1404 t4458 0 nch w=1u l=180n
M11720 t4458 nw1403 0 0 nch w=1u l=180n
M11721 t4456 nw1404 vdd vdd pch w=2u l=180n
M11722 t4456 t4455 vdd vdd pch w=2u l=180n
CT4459 t4459 0 0.1f
M11723 t4456 nw1404 t4459 0 nch w=1u l=180n
M11724 t4459 t4455 0 0 nch w=1u l=180n
M11725 t4457 nw1403 vdd vdd pch w=2u l=180n
M11726 t4457 t4455 vdd vdd pch w=2u l=180n
CT4460 t4460 0 0.1f
M11727 t4457 nw1403 t4460 0 nch w=1u l=180n
M11728 t4460 t4455 0 0 nch w=1u l=180n
M11729 nw1405 t4456 vdd vdd pch w=2u l=180n
M11730 nw1405 t4457 vdd vdd pch w=2u l=180n
CT4461 t4461 0 0.1f
M11731 nw1405 t4456 t4461 0 nch w=1u l=180n
M11732 t4461 t4457 0 0 nch w=1u l=180n
Cnw1405 nw1405 0 2f
M11733 nw1406 nw256 vdd vdd pch w=2u l=180n
M11734 nw1406 nw1331 vdd vdd pch w=2u l=180n
CT4462 t4462 0 0.1f
M11735 nw1406 nw256 t4462 0 nch w=1u l=180n
M11736 t4462 nw1331 0 0 nch w=1u l=180n
Cnw1406 nw1406 0 2f
M11737 nw1407 nw1404 vdd vdd pch w=2u l=180n
M11738 nw1407 nw1403 vdd vdd pch w=2u l=180n
CT4463 t4463 0 0.1f
M11739 nw1407 nw1404 t4463 0 nch w=1u l=180n
M11740 t4463 nw1403 0 0 nch w=1u l=180n
Cnw1407 nw1407 0 2f
M11741 nw1408 nw1406 vdd vdd pch w=2u l=180n
M11742 nw1408 nw1407 vdd vdd pch w=2u l=180n
CT4464 t4464 0 0.1f
M11743 nw1408 nw1406 t4464 0 nch w=1u l=180n
M11744 t4464 nw1407 0 0 nch w=1u l=180n
Cnw1408 nw1408 0 2f
CT4465 t4465 0 0.1f
M11745 t4465 nw1 vdd vdd pch w=2u l=180n
M11746 t4465 nw1 0 0 nch w=1u l=180n
M11747 np0 t4465 vdd vdd pch w=2u l=180n
M11748 np0 t4465 0 0 nch w=1u l=180n
Cnp0 np0 0 2f
CT4466 t4466 0 0.1f
M11749 t4466 nw257 vdd vdd pch w=2u l=180n
M11750 t4466 nw257 0 0 nch w=1u l=180n
M11751 np1 t4466 vdd vdd pch w=2u l=180n
M11752 np1 t4466 0 0 nch w=1u l=180n
Cnp1 np1 0 2f
CT4467 t4467 0 0.1f
M11753 t4467 nw331 vdd vdd pch w=2u l=180n
M11754 t4467 nw331 0 0 nch w=1u l=180n
M11755 np2 t4467 vdd vdd pch w=2u l=180n
M11756 np2 t4467 0 0 nch w=1u l=180n
Cnp2 np2 0 2f
CT4468 t4468 0 0.1f
M11757 t4468 nw408 vdd vdd pch w=2u l=180n
M11758 t4468 nw408 0 0 nch w=1u l=180n
M11759 np3 t4468 vdd vdd pch w=2u l=180n
M11760 np3 t4468 0 0 nch w=1u l=180n
Cnp3 np3 0 2f
CT4469 t4469 0 0.1f
M11761 t4469 nw485 vdd vdd pch w=2u l=180n
M11762 t4469 nw485 0 0 nch w=1u l=180n
M11763 np4 t4469 vdd vdd pch w=2u l=180n
M11764 np4 t4469 0 0 nch w=1u l=180n
Cnp4 np4 0 2f
CT4470 t4470 0 0.1f
M11765 t4470 nw562 vdd vdd pch w=2u l=180n
M11766 t4470 nw562 0 0 nch w=1u l=180n
M11767 np5 t4470 vdd vdd pch w=2u l=180n
M11768 np5 t4470 0 0 nch w=1u l=180n
Cnp5 np5 0 2f
CT4471 t4471 0 0.1f
M11769 t4471 nw639 vdd vdd pch w=2u l=180n
M11770 t4471 nw639 0 0 nch w=1u l=180n
M11771 np6 t4471 vdd vdd pch w=2u l=180n
M11772 np6 t4471 0 0 nch w=1u l=180n
Cnp6 np6 0 2f
CT4472 t4472 0 0.1f
M11773 t4472 nw716 vdd vdd pch w=2u l=180n
M11774 t4472 nw716 0 0 nch w=1u l=180n
M11775 np7 t4472 vdd vdd pch w=2u l=180n
M11776 np7 t4472 0 0 nch w=1u l=180n
Cnp7 np7 0 2f
CT4473 t4473 0 0.1f
M11777 t4473 nw793 vdd vdd pch w=2u l=180n
M11778 t4473 nw793 0 0 nch w=1u l=180n
M11779 np8 t4473 vdd vdd pch w=2u l=180n
M11780 np8 t4473 0 0 nch w=1u l=180n
Cnp8 np8 0 2f
CT4474 t4474 0 0.1f
M11781 t4474 nw870 vdd vdd pch w=2u l=180n
M11782 t4474 nw870 0 0 nch w=1u l=180n
M11783 np9 t4474 vdd vdd pch w=2u l=180n
M11784 np9 t4474 0 0 nch w=1u l=180n
Cnp9 np9 0 2f
CT4475 t4475 0 0.1f
M11785 t4475 nw947 vdd vdd pch w=2u l=180n
M11786 t4475 nw947 0 0 nch w=1u l=180n
M11787 np10 t4475 vdd vdd pch w=2u l=180n
M11788 np10 t4475 0 0 nch w=1u l=180n
Cnp10 np10 0 2f
CT4476 t4476 0 0.1f
M11789 t4476 nw1024 vdd vdd pch w=2u l=180n
M11790 t4476 nw1024 0 0 nch w=1u l=180n
M11791 np11 t4476 vdd vdd pch w=2u l=180n
M11792 np11 t4476 0 0 nch w=1u l=180n
Cnp11 np11 0 2f
CT4477 t4477 0 0.1f
M11793 t4477 nw1101 vdd vdd pch w=2u l=180n
M11794 t4477 nw1101 0 0 nch w=1u l=180n
M11795 np12 t4477 vdd vdd pch w=2u l=180n
M11796 np12 t4477 0 0 nch w=1u l=180n
Cnp12 np12 0 2f
CT4478 t4478 0 0.1f
M11797 t4478 nw1178 vdd vdd pch w=2u l=180n
M11798 t4478 nw1178 0 0 nch w=1u l=180n
M11799 np13 t4478 vdd vdd pch w=2u l=180n
M11800 np13 t4478 0 0 nch w=1u l=180n
Cnp13 np13 0 2f
CT4479 t4479 0 0.1f
M11801 t4479 nw1255 vdd vdd pch w=2u l=180n
M11802 t4479 nw1255 0 0 nch w=1u l=180n
M11803 np14 t4479 vdd vdd pch w=2u l=180n
M11804 np14 t4479 0 0 nch w=1u l=180n
Cnp14 np14 0 2f
CT4480 t4480 0 0.1f
M11805 t4480 nw1332 vdd vdd pch w=2u l=180n
M11806 t4480 nw1332 0 0 nch w=1u l=180n
M11807 np15 t4480 vdd vdd pch w=2u l=180n
M11808 np15 t4480 0 0 nch w=1u l=180n
Cnp15 np15 0 2f
CT4481 t4481 0 0.1f
M11809 t4481 nw1335 vdd vdd pch w=2u l=180n
M11810 t4481 nw1335 0 0 nch w=1u l=180n
M11811 np16 t4481 vdd vdd pch w=2u l=180n
M11812 np16 t4481 0 0 nch w=1u l=180n
Cnp16 np16 0 2f
CT4482 t4482 0 0.1f
M11813 t4482 nw1340 vdd vdd pch w=2u l=180n
M11814 t4482 nw1340 0 0 nch w=1u l=180n
M11815 np17 t4482 vdd vdd pch w=2u l=180n
M11816 np17 t4482 0 0 nch w=1u l=180n
Cnp17 np17 0 2f
CT4483 t4483 0 0.1f
M11817 t4483 nw1345 vdd vdd pch w=2u l=180n
M11818 t4483 nw1345 0 0 nch w=1u l=180n
M11819 np18 t4483 vdd vdd pch w=2u l=180n
M11820 np18 t4483 0 0 nch w=1u l=180n
Cnp18 np18 0 2f
CT4484 t4484 0 0.1f
M11821 t4484 nw1350 vdd vdd pch w=2u l=180n
M11822 t4484 nw1350 0 0 nch w=1u l=180n
M11823 np19 t4484 vdd vdd pch w=2u l=180n
M11824 np19 t4484 0 0 nch w=1u l=180n
Cnp19 np19 0 2f
CT4485 t4485 0 0.1f
M11825 t4485 nw1355 vdd vdd pch w=2u l=180n
M11826 t4485 nw1355 0 0 nch w=1u l=180n
M11827 np20 t4485 vdd vdd pch w=2u l=180n
M11828 np20 t4485 0 0 nch w=1u l=180n
Cnp20 np20 0 2f
CT4486 t4486 0 0.1f
M11829 t4486 nw1360 vdd vdd pch w=2u l=180n
M11830 t4486 nw1360 0 0 nch w=1u l=180n
M11831 np21 t4486 vdd vdd pch w=2u l=180n
M11832 np21 t4486 0 0 nch w=1u l=180n
Cnp21 np21 0 2f
CT4487 t4487 0 0.1f
M11833 t4487 nw1365 vdd vdd pch w=2u l=180n
M11834 t4487 nw1365 0 0 nch w=1u l=180n
M11835 np22 t4487 vdd vdd pch w=2u l=180n
M11836 np22 t4487 0 0 nch w=1u l=180n
Cnp22 np22 0 2f
CT4488 t4488 0 0.1f
M11837 t4488 nw1370 vdd vdd pch w=2u l=180n
M11838 t4488 nw1370 0 0 nch w=1u l=180n
M11839 np23 t4488 vdd vdd pch w=2u l=180n
M11840 np23 t4488 0 0 nch w=1u l=180n
Cnp23 np23 0 2f
CT4489 t4489 0 0.1f
M11841 t4489 nw1375 vdd vdd pch w=2u l=180n
M11842 t4489 nw1375 0 0 nch w=1u l=180n
M11843 np24 t4489 vdd vdd pch w=2u l=180n
M11844 np24 t4489 0 0 nch w=1u l=180n
Cnp24 np24 0 2f
CT4490 t4490 0 0.1f
M11845 t4490 nw1380 vdd vdd pch w=2u l=180n
M11846 t4490 nw1380 0 0 nch w=1u l=180n
M11847 np25 t4490 vdd vdd pch w=2u l=180n
M11848 np25 t4490 0 0 nch w=1u l=180n
Cnp25 np25 0 2f
CT4491 t4491 0 0.1f
M11849 t4491 nw1385 vdd vdd pch w=2u l=180n
M11850 t4491 nw1385 0 0 nch w=1u l=180n
M11851 np26 t4491 vdd vdd pch w=2u l=180n
M11852 np26 t4491 0 0 nch w=1u l=180n
Cnp26 np26 0 2f
CT4492 t4492 0 0.1f
M11853 t4492 nw1390 vdd vdd pch w=2u l=180n
M11854 t4492 nw1390 0 0 nch w=1u l=180n
M11855 np27 t4492 vdd vdd pch w=2u l=180n
M11856 np27 t4492 0 0 nch w=1u l=180n
Cnp27 np27 0 2f
CT4493 t4493 0 0.1f
M11857 t4493 nw1395 vdd vdd pch w=2u l=180n
M11858 t4493 nw1395 0 0 nch w=1u l=180n
M11859 np28 t4493 vdd vdd pch w=2u l=180n
M11860 np28 t4493 0 0 nch w=1u l=180n
Cnp28 np28 0 2f
CT4494 t4494 0 0.1f
M11861 t4494 nw1400 vdd vdd pch w=2u l=180n
M11862 t4494 nw1400 0 0 nch w=1u l=180n
M11863 np29 t4494 vdd vdd pch w=2u l=180n
M11864 np29 t4494 0 0 nch w=1u l=180n
Cnp29 np29 0 2f
CT4495 t4495 0 0.1f
M11865 t4495 nw1405 vdd vdd pch w=2u l=180n
M11866 t4495 nw1405 0 0 nch w=1u l=180n
M11867 np30 t4495 vdd vdd pch w=2u l=180n
M11868 np30 t4495 0 0 nch w=1u l=180n
Cnp30 np30 0 2f
CT4496 t4496 0 0.1f
M11869 t4496 nw1408 vdd vdd pch w=2u l=180n
M11870 t4496 nw1408 0 0 nch w=1u l=180n
M11871 np31 t4496 vdd vdd pch w=2u l=180n
M11872 np31 t4496 0 0 nch w=1u l=180n
Cnp31 np31 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: np0 np1 np2 np3 np4 np5 np6 np7 np8 np9 np10 np11 np12 np13 np14 np15 np16 np17 np18 np19 np20 np21 np22 np23 np24 np25 np26 np27 np28 np29 np30 np31
.end
